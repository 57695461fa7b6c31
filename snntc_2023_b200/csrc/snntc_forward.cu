// SNN-TC forward (SnnFc / SnnCv) for sm_100a: gather -> sort in shared memory -> sorted walk.
//
// One CTA takes a group of rows (dense samples or conv receptive fields, gathered straight from the
// NHWC image with MAX outside it), packs each element as (sortable value bits << 32 | source index),
// sorts every row of the group in shared memory with a bitonic network that needs no power-of-two
// padding, and then lets each warp walk one row for 32*JPT outputs: lanes span consecutive output
// columns so every weight-row read is one coalesced 128-byte line. The walk keeps the running
// sum(w)-theta and sum(w*x) per output in registers in sorted order, bias first, and applies the
// division-free causality test of the reference kernel (snntc/snnfc_kernels.cu.cc:33-69).
#include "snntc_common.cuh"

namespace snntc {

namespace {

constexpr int kFwdThreads = 256;
constexpr int kFwdWarps = kFwdThreads / 32;
constexpr int kMaxRowsPerPass = 32;
constexpr int kUnroll = 4;

typedef unsigned long long u64;

__device__ __forceinline__ void compare_exchange(u64* a, u64* b) {
  u64 va = *a, vb = *b;
  if (va > vb) { *a = vb; *b = va; }
}

// One step of the walk for one output: test "fire before consuming x", else consume (x, wv).
__device__ __forceinline__ void walk_step(float x, float wv, float& wsum, float& ysum, bool& armed, bool& live) {
  if (live) {
    float wa = fabsf(wsum);
    float ya = wsum < 0.f ? -ysum : ysum;
    if (armed && ya <= x * wa) {
      live = false;  // spike lies in (previous input, x]: keep the sums as they are
    } else {
      wsum += wv;
      ysum = fmaf(x, wv, ysum);
      wa = fabsf(wsum);
      ya = wsum < 0.f ? -ysum : ysum;
      armed = ya > x * wa;
    }
  }
}

template <int JPT>
__device__ __forceinline__ void walk_row(const Geometry& g, const u64* __restrict__ keys, int nvalid,
                                         const float* __restrict__ w, int jbase, int lane,
                                         float* __restrict__ y_row, float* __restrict__ inv_row) {
  const int J = g.J;
  int jl[JPT];
  bool jok[JPT];
  float wsum[JPT], ysum[JPT];
  bool armed[JPT], live[JPT];
#pragma unroll
  for (int m = 0; m < JPT; ++m) {
    int j = jbase + lane + 32 * m;
    jok[m] = j < J;
    jl[m] = jok[m] ? j : J - 1;
    wsum[m] = -g.theta;
    ysum[m] = 0.f;
    armed[m] = false;
    live[m] = true;
    if (g.has_bias) {  // the bias input (value biasvolt, weight row I) is always consumed first
      float wb = __ldg(w + (size_t)g.I * J + jl[m]);
      wsum[m] += wb;
      ysum[m] = g.biasvolt * wb;
      float wa = fabsf(wsum[m]);
      float ya = wsum[m] < 0.f ? -ysum[m] : ysum[m];
      armed[m] = ya > wa * g.biasvolt;
    }
  }

  int k = 0;
  bool all_done = false;
  for (; k + kUnroll <= nvalid && !all_done; k += kUnroll) {
    float xs[kUnroll];
    float wv[kUnroll][JPT];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      u64 e = keys[k + u];
      xs[u] = sortable_to_float((uint32_t)(e >> 32));
      const float* wrow = w + (size_t)(uint32_t)e * J;
#pragma unroll
      for (int m = 0; m < JPT; ++m) wv[u][m] = __ldg(wrow + jl[m]);
    }
    bool any_live = false;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int m = 0; m < JPT; ++m) walk_step(xs[u], wv[u][m], wsum[m], ysum[m], armed[m], live[m]);
    }
#pragma unroll
    for (int m = 0; m < JPT; ++m) any_live |= live[m];
    all_done = !__any_sync(0xffffffffu, any_live);
  }
  if (!all_done) {
    for (; k < nvalid; ++k) {
      u64 e = keys[k];
      float x = sortable_to_float((uint32_t)(e >> 32));
      const float* wrow = w + (size_t)(uint32_t)e * J;
#pragma unroll
      for (int m = 0; m < JPT; ++m) {
        float wv = __ldg(wrow + jl[m]);
        walk_step(x, wv, wsum[m], ysum[m], armed[m], live[m]);
      }
    }
  }

#pragma unroll
  for (int m = 0; m < JPT; ++m) {
    float yv = g.maxv, iv = 0.f;
    if (armed[m]) {
      iv = __fdividef(1.0f, wsum[m]);
      yv = ysum[m] * iv;
      if (yv >= g.maxv) { yv = g.maxv; iv = 0.f; }
    }
    if (jok[m]) {
      int j = jbase + lane + 32 * m;
      y_row[j] = yv;
      inv_row[j] = iv;
    }
  }
}

template <int JPT>
__global__ void __launch_bounds__(kFwdThreads)
snn_forward_kernel(const Geometry g, const float* __restrict__ x, const float* __restrict__ w,
                   float* __restrict__ out, int rows_per_pass, int npad, int log2_half) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  u64* keys = reinterpret_cast<u64*>(smem_raw);
  __shared__ int s_nvalid[kMaxRowsPerPass];

  const int I = g.I, J = g.J, R = g.R;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int num_groups = (R + rows_per_pass - 1) / rows_per_pass;
  const int jchunks = (J + 32 * JPT - 1) / (32 * JPT);
  const uint32_t max_key = float_to_sortable(g.maxv - 0.1f);
  float* __restrict__ y_out = out;
  float* __restrict__ inv_out = out + (size_t)R * J;

  for (int group = blockIdx.x; group < num_groups; group += gridDim.x) {
    const int r0 = group * rows_per_pass;
    const int nrows = min(rows_per_pass, R - r0);

    // ---- 1. gather rows into shared memory as sortable (value, index) pairs
    for (int rr = warp; rr < nrows; rr += kFwdWarps) {
      const int r = r0 + rr;
      u64* krow = keys + (size_t)rr * I;
      if (!g.is_conv) {
        const float* xr = x + (size_t)r * I;
        for (int i = lane; i < I; i += 32)
          krow[i] = ((u64)float_to_sortable(__ldg(xr + i)) << 32) | (uint32_t)i;
      } else {
        const int nw = r % g.Nw;
        const int t = r / g.Nw;
        const int nh = t % g.Nh;
        const int b = t / g.Nh;
        const int h0 = nh * g.Sh - g.pad_top, w0 = nw * g.Sw - g.pad_left;
        for (int i = lane; i < I; i += 32) {
          const int tap = i / g.C, c = i - tap * g.C;
          const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
          const int h = h0 + kh, ww = w0 + kw;
          float v = g.maxv;
          if (h >= 0 && h < g.H && ww >= 0 && ww < g.W)
            v = __ldg(x + (((size_t)b * g.H + h) * g.W + ww) * g.C + c);
          krow[i] = ((u64)float_to_sortable(v) << 32) | (uint32_t)i;
        }
      }
    }
    __syncthreads();

    // ---- 2. bitonic sort of every row; every compare-exchange moves the smaller key to the lower
    // index, so virtual +inf elements at positions >= I never move and need no storage.
    {
      const int half = npad >> 1;
      const int total = nrows * half;
      for (int k = 2; k <= npad; k <<= 1) {
        const int hk = k >> 1;
        for (int t = tid; t < total; t += kFwdThreads) {
          const int rr = t >> log2_half, q = t & (half - 1);
          const int o = q & (hk - 1);
          const int base = (q - o) << 1;
          const int i = base + o, p = base + k - 1 - o;
          if (p < I) compare_exchange(keys + (size_t)rr * I + i, keys + (size_t)rr * I + p);
        }
        __syncthreads();
        for (int j = hk >> 1; j >= 1; j >>= 1) {
          for (int t = tid; t < total; t += kFwdThreads) {
            const int rr = t >> log2_half, q = t & (half - 1);
            const int o = q & (j - 1);
            const int i = ((q - o) << 1) + o, p = i + j;
            if (p < I) compare_exchange(keys + (size_t)rr * I + i, keys + (size_t)rr * I + p);
          }
          __syncthreads();
        }
      }
    }

    // ---- 3. inputs above MAX-0.1 never spike: the walk stops at the first of them
    if (tid < nrows) {
      const u64* krow = keys + (size_t)tid * I;
      int lo = 0, hi = I;
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if ((uint32_t)(krow[mid] >> 32) <= max_key) lo = mid + 1; else hi = mid;
      }
      s_nvalid[tid] = lo;
    }
    __syncthreads();

    // ---- 4. walk
    const int items = nrows * jchunks;
    for (int item = warp; item < items; item += kFwdWarps) {
      const int rr = item / jchunks, jc = item - rr * jchunks;
      const size_t r = (size_t)(r0 + rr);
      walk_row<JPT>(g, keys + (size_t)rr * I, s_nvalid[rr], w, jc * 32 * JPT, lane, y_out + r * J, inv_out + r * J);
    }
    __syncthreads();
  }
}

int pick_rows_per_pass(const Geometry& g, const LaunchInfo& li) {
  const size_t per_row = (size_t)g.I * sizeof(u64);
  const size_t budget = (size_t)li.max_smem_optin - 1024;
  if (per_row > budget) return 0;
  size_t soft = 96 * 1024;  // leave room for two CTAs per SM when rows are short
  int rt = (int)((soft > per_row ? soft : per_row) / per_row);
  if (rt > kMaxRowsPerPass) rt = kMaxRowsPerPass;
  // do not starve the grid: aim for at least ~2 groups per SM
  long want = ((long)g.R + 2L * li.num_sms - 1) / (2L * li.num_sms);
  if (want < 1) want = 1;
  if (rt > want) rt = (int)want;
  if (rt < 1) rt = 1;
  return rt;
}

template <int JPT>
int launch_t(const Geometry& g, const float* x, const float* w, float* out, const LaunchInfo& li, cudaStream_t s) {
  const int rt = pick_rows_per_pass(g, li);
  if (rt == 0) return E_UNSUPPORTED;
  int npad = 1, log2n = 0;
  while (npad < g.I) { npad <<= 1; ++log2n; }
  const int log2_half = log2n > 0 ? log2n - 1 : 0;
  const size_t smem = (size_t)rt * g.I * sizeof(u64);
  auto kern = snn_forward_kernel<JPT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)li.max_smem_optin - 1024) != cudaSuccess)
    return E_CUDA;
  const int groups = (g.R + rt - 1) / rt;
  int ctas_per_sm = (int)(((size_t)li.max_smem_optin) / (smem + 2048));
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  if (ctas_per_sm > 4) ctas_per_sm = 4;
  int grid = li.num_sms * ctas_per_sm;
  if (grid > groups) grid = groups;
  kern<<<grid, kFwdThreads, smem, s>>>(g, x, w, out, rt, npad < 2 ? 2 : npad, log2_half);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

}  // namespace

size_t forward_workspace_bytes(const Geometry&) { return 0; }

int launch_forward(const Geometry& g, const float* x, const float* w, float* out, void*, size_t,
                   const LaunchInfo& li, cudaStream_t s) {
  if (g.J <= 32) return launch_t<1>(g, x, w, out, li, s);
  if (g.J <= 64) return launch_t<2>(g, x, w, out, li, s);
  return launch_t<4>(g, x, w, out, li, s);
}

}  // namespace snntc
