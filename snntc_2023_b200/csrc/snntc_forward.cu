// SNN-TC forward (SnnFc / SnnCv) for sm_100a: sorted lists of the inputs that can spike -> sorted walk.
//
// Rows are dense samples or conv receptive fields (gathered straight from the NHWC image with MAX
// outside it). A scratch buffer of sorted lists in global memory -- per row the inputs at or below MAX-0.1 as
// (value, element offset of the weight row), ascending -- joins two stages:
//   1. the lists. Stride-1 convolutions up to 3x3 on 16 to 512 channels: per-pixel sort and two levels of
//      merging (snntc_lists.cu). Rows of at most 256 inputs: a sorting network in registers, one warp per row
//      (snntc_lists.cu). Everything else, here: one warp per row gathers the row into shared memory as 32-bit
//      sortable value bits plus a 16-bit source index (conv rows find their taps through a per-CTA table, with
//      predicated loads and no divergent branch), rebases the keys to the row's smallest, counts the 8-bit digits
//      that the row's range needs and runs a stable least-significant-digit radix sort over those digits only (a
//      last digit of one or two bits is a ballot split); rows too long for two shared-memory buffers fall back
//      to a CTA-wide in-place bitonic network;
//   2. the walk (walk kernels): every warp takes (row, block of outputs) items and walks the row's list, which it
//      stages through shared memory 32 entries at a time. The running sum(w)-theta and sum(w*x) stay in
//      registers, in sorted order, bias first, with the arithmetic of the reference kernel
//      (snntc/snnfc_kernels.cu.cc:33-69); the causality test is the sign of q = ysum - x*wsum per step -- one FMA
//      per output, the lane's smallest q as an integer, one warp vote -- backed by the reference's exact
//      division-free comparisons whenever it turns non-positive in any lane (see walk_row). Three layouts of a
//      lane's outputs: a pair in one 64-bit register (walk_row2, fan-out <= 64), 2 or 4 consecutive outputs read
//      by one 8/16-byte load, or outputs lane + 32*m (odd fan-out, unaligned weights).
#include "snntc_common.cuh"

#include <limits.h>
#include <math_constants.h>

namespace snntc {

namespace {

constexpr int kFwdThreads = 256;
constexpr int kFwdWarps = kFwdThreads / 32;

typedef unsigned long long u64;

// Index of this warp in its CTA, broadcast from lane 0: the value is the same for all 32 lanes anyway, but only
// a shuffle from a fixed lane lets the compiler treat everything derived from it (row numbers, list lengths,
// loop bounds) as warp-uniform, and with that it drops the divergence check in front of every warp vote.
__device__ __forceinline__ int uniform_warp_index() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

__device__ __forceinline__ float key_value(u64 e) { return sortable_to_float((uint32_t)(e >> 32)); }

// ------------------------------------------------------------------------------------------- walk

// "ysum/wsum > c" without a division, as the reference evaluates it after consuming input c
// (snntc/snnfc_kernels.cu.cc:53-55)
__device__ __forceinline__ bool ratio_gt(float ysum, float wsum, float c) {
  const float wa = fabsf(wsum);
  const float ya = wsum < 0.f ? -ysum : ysum;
  return ya > c * wa;
}
// "ysum/wsum <= c" (snntc/snnfc_kernels.cu.cc:46-48)
__device__ __forceinline__ bool ratio_le(float ysum, float wsum, float c) {
  const float wa = fabsf(wsum);
  const float ya = wsum < 0.f ? -ysum : ysum;
  return ya <= c * wa;
}

// Smallest of three float bit patterns compared as signed integers. For the sign test of the walk that is all
// that is needed: the result is <= 0 exactly when one of the floats is negative, -0 or +0 (negative floats are
// negative integers, +0 is 0, positive floats and NaN patterns with a clear sign bit are positive integers).
__device__ __forceinline__ int imin3(int a, int b, int c) { return min(min(a, b), c); }

// How close to zero q = ysum - x*wsum may be before the sign of q stops deciding. The reference compares
// ysum against the ROUNDED product x*wsum (ratio_gt / ratio_le below), so it can see "ysum <= x*wsum" while the
// exact difference is still positive by up to half an ulp of the product, and the other way round for the test
// against the previous input. The walk therefore hands a step over to the reference's comparisons whenever
// q <= tol, tol = 2^-21 * |x| * (|theta| + B), B = sum of g.wbound[] >= sum_i |w_ij| for every output j: |wsum| never
// exceeds |theta| + B, so tol is at least eight times the largest rounding error of the product, and small enough
// to be met by chance about once in 10^5 output steps. Compared as integers: tol >= +0, negative q are negative.
__device__ __forceinline__ float walk_tolerance_base(const Geometry& g) {
  const int lane = threadIdx.x & 31;
  float b = lane < g.wbound_n ? __ldg(g.wbound + lane) : 0.f;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) b += __shfl_xor_sync(0xffffffffu, b, d);
  return 4.76837158203125e-7f * (fabsf(g.theta) + b) * 1.0001f;   // (a little slack for the rounding of the sums)
}

// bound[blockIdx.x] = sum over this CTA's weight rows of max_j |w_ij|: summed over the CTAs an upper bound on every
// column's sum of magnitudes. rows = I + bias row; CTA c takes rows [c * rows_per_cta, (c + 1) * rows_per_cta).
constexpr int kBoundMaxCtas = 32;
__global__ void __launch_bounds__(256)
snn_wbound_kernel(const float* __restrict__ w, int rows, int J, int rows_per_cta, float* __restrict__ bound) {
  __shared__ float part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = blockIdx.x * rows_per_cta;
  float acc = 0.f;                                     // lane 0: sum of the row maxima of this warp's rows
  for (int r = r0 + warp; r < min(rows, r0 + rows_per_cta); r += 8) {
    const float* wr = w + (size_t)r * J;
    float m = 0.f;
    for (int j = lane; j < J; j += 32) m = fmaxf(m, fabsf(__ldg(wr + j)));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    acc += m;
  }
  if (lane == 0) part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += part[k];
    bound[blockIdx.x] = t;
  }
}

// Number of list entries whose input value lies strictly below y: the causal-set size of an output that fired
// at y (every consumed input is below the spike value, every other one is not). Binary search, one thread.
__device__ __forceinline__ int entries_below(const WalkEntry* __restrict__ ents, int n, float y) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__uint_as_float(__ldcg(ents + mid).x) < y) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One warp walks one row for 32*JPT outputs. Let q_k = ysum - x_k*wsum be taken just before input k is
// consumed. The reference fires at step k when "ysum/wsum > previous input" and "ysum/wsum <= x_k", i.e.
// sign(wsum)*q_{k-1} > 0 >= sign(wsum)*q_k (q_{k-1} re-evaluated with the sums of step k, which leaves its
// value unchanged). With a positive denominator -- the only case in which an output of sorted inputs at or
// above the bias input can fire -- that is the first k with q_k <= 0. The loop therefore computes one extra FMA
// per output and step (q, with its exact sign), takes the smallest q of the lane and one warp vote; only when
// some lane sees q <= 0 does the warp evaluate the reference's own rounded, division-free tests
// (snntc/snnfc_kernels.cu.cc:46-55) for its live outputs, so the decision is the reference's, an exact tie
// (q == 0) included. An output whose q is not positive but which the reference test did not fire -- q within an
// ulp of zero, or a NEGATIVE denominator, which inputs below the bias input can produce and for which the
// reference fires on the way back up through zero -- makes the lane "sticky": the exact tests run again at
// the next step whatever q is, until no live output of the lane is in that state any more.
template <int JPT, int CH, bool FULL, bool VECW, bool STAGE>
__device__ __forceinline__ void walk_row(const Geometry& g, const WalkEntry* __restrict__ ents, int nvalid,
                                         const float* __restrict__ w, int jbase, int lane,
                                         float* __restrict__ y_row, float* __restrict__ inv_row,
                                         WalkEntry* __restrict__ sbuf) {
  const int J = g.J;
  int jl[JPT];
  bool jok[JPT];
  float wsum[JPT], ysum[JPT], wfin[JPT], yfin[JPT];
  int livemask[JPT];
#pragma unroll
  for (int m = 0; m < JPT; ++m) {
    // VECW: a lane owns JPT consecutive outputs and reads them with 8- or 16-byte loads (J % JPT == 0,
    // so a lane is wholly inside or wholly outside the row); otherwise outputs lane + 32*m, 4-byte loads
    const int j = VECW ? jbase + JPT * lane + m : jbase + lane + 32 * m;
    jok[m] = FULL || j < J;
    jl[m] = jok[m] ? j : (VECW ? J - JPT + m : J - 1);
    wsum[m] = -g.theta;
    ysum[m] = 0.f;
    if (g.has_bias) {  // the bias input (value biasvolt, weight row I) is always consumed first
      const float wb = __ldg(w + (size_t)g.I * J + jl[m]);
      wsum[m] += wb;
      ysum[m] = g.biasvolt * wb;
    }
    wfin[m] = wsum[m];
    yfin[m] = ysum[m];
    livemask[m] = -1;
  }
  // Without bias the sums start at (-theta, 0), for which "ysum/wsum > c" is false for every c >= 0, so the
  // first step needs no special case; with bias the previous input is the bias input itself.
  float xprev = g.has_bias ? g.biasvolt : 0.f;
  int sticky = INT_MAX;   // INT_MIN while some live output of this lane must be tested exactly at the next step
  const float tolbase = walk_tolerance_base(g);
  int qlim = 0;           // bits of the largest q that still goes to the exact tests (see walk_tolerance_base)

  const float* wl = w + (VECW ? jl[0] : (FULL ? jbase + lane : 0));
  // VECW: addressed by a 32-bit element offset from the (uniform) weight base, widened before the scaling to
  // bytes -- measured faster than a 64-bit per-lane pointer plus the entry's offset
  const unsigned lane_off = (unsigned)jl[0];
  const char* wbase = reinterpret_cast<const char*>(w);
  auto load_weights = [&](unsigned eoff, float (&wv)[JPT]) {
    const float* wrow = wl + eoff;
    if constexpr (VECW && JPT == 8) {
      const float4* p4 = reinterpret_cast<const float4*>(wbase + (size_t)(eoff + lane_off) * 4u);
      const float4 v = __ldg(p4), v2 = __ldg(p4 + 1);
      wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
      wv[4] = v2.x; wv[5] = v2.y; wv[6] = v2.z; wv[7] = v2.w;
    } else if constexpr (VECW && JPT == 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(wbase + (size_t)(eoff + lane_off) * 4u));
      wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
    } else if constexpr (VECW && JPT == 2) {
      const float2 v = __ldg(reinterpret_cast<const float2*>(wbase + (size_t)(eoff + lane_off) * 4u));
      wv[0] = v.x; wv[1] = v.y;
    } else {
#pragma unroll
      for (int m = 0; m < JPT; ++m) wv[m] = FULL ? __ldg(wrow + 32 * m) : __ldg(wrow + jl[m]);
    }
  };

  // one step for all JPT outputs of this lane: sign test, (rarely) exact test, then consume
  auto step = [&](const float x, const float xprev, const float (&wv)[JPT]) {
    int q[JPT];
#pragma unroll
    for (int m = 0; m < JPT; ++m) q[m] = __float_as_int(fmaf(-x, wsum[m], ysum[m]));
    int qmin;
    if constexpr (JPT == 1) qmin = min(q[0], sticky);
    else if constexpr (JPT == 2) qmin = imin3(q[0], q[1], sticky);
    else if constexpr (JPT == 4) qmin = imin3(imin3(q[0], q[1], q[2]), q[3], sticky);
    else qmin = imin3(imin3(q[0], q[1], q[2]), imin3(q[3], q[4], q[5]), imin3(q[6], q[7], sticky));
    if (__builtin_expect(__any_sync(0xffffffffu, qmin <= qlim), 0)) {
      // rare path: the reference's own rounded comparisons for the live outputs concerned (usually one of the
      // lane's outputs in one lane: skip the others with a warp-uniform test each)
      bool again = false;
#pragma unroll
      for (int m = 0; m < JPT; ++m) {
        if (JPT > 1 && !__any_sync(0xffffffffu, (q[m] <= qlim) | (sticky < 0))) continue;
        const bool live = livemask[m] != 0;
        const bool fire = live & ratio_gt(ysum[m], wsum[m], xprev) & ratio_le(ysum[m], wsum[m], x);
        if (fire) {
          livemask[m] = 0;  // spike lies in (previous input, x]: keep the sums aside ...
          wfin[m] = wsum[m];
          yfin[m] = ysum[m];
          // ... and park the running ones where q can never be non-positive again: with wsum = -inf,
          // q = ysum + x*inf = +inf at every later step
          wsum[m] = -CUDART_INF_F;
        }
        again |= live & !fire & (q[m] <= qlim);
      }
      sticky = again ? INT_MIN : INT_MAX;
    }
#pragma unroll
    for (int m = 0; m < JPT; ++m) {
      wsum[m] += wv[m];
      ysum[m] = fmaf(x, wv[m], ysum[m]);
    }
  };

  // One chunk of CH steps: entries, then their weight rows, then the arithmetic. `fetch(i)` returns entry i of
  // the part of the list at hand.
  bool all_done = false;
  auto check_done = [&]() {
    int any_live = 0;
#pragma unroll
    for (int m = 0; m < JPT; ++m) any_live |= livemask[m];
    all_done = !__any_sync(0xffffffffu, any_live != 0);
  };
  // `fetch2(i)` returns entries i and i+1 (i even) of the part of the list at hand as one 16-byte read.
  static_assert(CH % 2 == 0, "entries are fetched two at a time");
  auto chunk = [&](auto fetch2, int k0) {
    float xs[CH];
    float wv[CH][JPT];
#pragma unroll
    for (int u = 0; u < CH; u += 2) {
      const uint4 e2 = fetch2(k0 + u);
      xs[u] = __uint_as_float(e2.x);
      load_weights(e2.y, wv[u]);
      xs[u + 1] = __uint_as_float(e2.z);
      load_weights(e2.w, wv[u + 1]);
    }
    qlim = __float_as_int(tolbase * fmaxf(fabsf(xs[0]), fabsf(xs[CH - 1])));   // inputs ascend: |x| peaks at an end
#pragma unroll
    for (int u = 0; u < CH; ++u) step(xs[u], u == 0 ? xprev : xs[u > 0 ? u - 1 : 0], wv[u]);
    xprev = xs[CH - 1];   // the previous input is only read when an output is about to fire: no copy per step
  };
  auto single = [&](const WalkEntry e) {
    float wv[JPT];
    load_weights(e.y, wv);
    qlim = __float_as_int(tolbase * fabsf(__uint_as_float(e.x)));
    step(__uint_as_float(e.x), xprev, wv);
    xprev = __uint_as_float(e.x);
  };
  if constexpr (STAGE) {
    // The list goes through shared memory 32 entries at a time: one coalesced read per lane and block, issued a
    // whole block ahead, instead of one L2 round trip in front of every chunk; a step then reads its entry with
    // one broadcast shared-memory load. Two buffers of 32 entries per warp.
    WalkEntry pre = make_uint2(0u, 0u);
    if (lane < nvalid) pre = __ldcg(ents + lane);
    int b = 0;
    for (int base = 0; base < nvalid && !all_done; base += 32, b ^= 32) {
      sbuf[b + lane] = pre;
      __syncwarp();
      if (base + 32 + lane < nvalid) pre = __ldcg(ents + base + 32 + lane);
      const int nb = min(32, nvalid - base);
      const WalkEntry* cur = sbuf + b;
      auto fetch2 = [&](int i) { return *reinterpret_cast<const uint4*>(cur + i); };
      int kk = 0;
#pragma unroll 1
      for (; kk + CH <= nb; kk += CH) chunk(fetch2, kk);
      for (; kk < nb; ++kk) single(cur[kk]);
      check_done();   // one "has every output fired" vote per block
    }
  } else {
    int k = 0;
    for (; k + CH <= nvalid && !all_done; k += CH) {
      // list entries bypass L1: it is kept for the weights
      chunk([&](int i) { return __ldcg(reinterpret_cast<const uint4*>(ents + i)); }, k);
      check_done();
    }
    if (!all_done)
      for (; k < nvalid; ++k) single(__ldcg(ents + k));
  }

#pragma unroll
  for (int m = 0; m < JPT; ++m) {
    // an output that stopped has fired; one that consumed every input fires iff it is armed
    bool fired = true;
    float ws = wfin[m], ys = yfin[m];
    if (livemask[m]) {
      ws = wsum[m]; ys = ysum[m];
      fired = ratio_gt(ys, ws, xprev);
    }
    float yv = g.maxv, iv = 0.f;
    if (fired) {
      iv = __fdividef(1.0f, ws);
      yv = ys * iv;
      if (yv >= g.maxv) { yv = g.maxv; iv = 0.f; }
    }
    if (jok[m]) {
      const int j = VECW ? jbase + JPT * lane + m : jbase + lane + 32 * m;
      y_row[j] = yv;
      if (inv_row != nullptr) inv_row[j] = iv;
      if (g.khist != nullptr) atomicAdd(g.khist + (yv < g.maxv ? entries_below(ents, nvalid, yv) : g.I + 1), 1);
    }
  }
}

// ---- two outputs per 64-bit register ---------------------------------------------------------------
// sm_100 has two-lane FP32 add / sub / fma on 64-bit register pairs: one issue slot, two results, each
// rounded exactly like the scalar instruction. A pair holds outputs (j, j+1) of one lane.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void unpack2i(uint64_t v, int& lo, int& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// walk_row with the outputs of a lane held as JP pairs (j, j+1), j = jbase + 2*lane + 64*m: the three
// FP32 operations of a step (q, the weight sum, the weighted sum) are one packed instruction per pair and
// a weight-row read is one 8-byte load per pair. The weight sum is carried NEGATED (nws = theta - sum w), so
// that q = fma(x, nws, ysum) needs no negated copy of x; negation is exact, so every value is bit for bit the
// scalar walk's -- except the sign of an exactly cancelled sum (+0 on both sides), which is why the sum is
// read back as 0 - nws: 1/(+0) = +inf clamps to "no spike", 1/(-0) would not. Requires J even and the
// weights 8-byte aligned.
// WS: the weights of this warp's 64 outputs sit in shared memory as [fan-in row][64] (see snn_walk2_smemw_kernel);
// `ws_lane` is the shared-memory byte address of this lane's pair in row 0 and `wmul` = 256 / J (J = 64, 128 or 256): a
// list entry's element offset (source index * J) times wmul is the row's byte offset in the slice -- one integer
// multiply-add on the FMA pipe per weight read. JP == 1 only.
template <int JP, int CH, bool FULL, bool STAGE, bool WS = false>
__device__ __forceinline__ void walk_row2(const Geometry& g, const WalkEntry* __restrict__ ents, int nvalid,
                                          const float* __restrict__ w, int jbase, int lane,
                                          float* __restrict__ y_row, float* __restrict__ inv_row,
                                          WalkEntry* __restrict__ sbuf, unsigned ws_lane = 0u, unsigned wmul = 0u) {
  static_assert(!WS || JP == 1, "weights in shared memory: one output pair per lane");
  const int J = g.J;
  int jl[JP];
  bool jok[JP];
  uint64_t nws[JP], ys[JP];
  float wfin[2 * JP], yfin[2 * JP];
  int live[2 * JP];
#pragma unroll
  for (int m = 0; m < JP; ++m) {
    const int j = jbase + 2 * lane + 64 * m;
    jok[m] = FULL || j < J;
    jl[m] = jok[m] ? j : J - 2;
    float n0 = g.theta, n1 = g.theta, y0 = 0.f, y1 = 0.f;
    if (g.has_bias) {  // the bias input (value biasvolt, weight row I) is always consumed first
      const float2 wb = __ldg(reinterpret_cast<const float2*>(w + (size_t)g.I * J + jl[m]));
      n0 -= wb.x; n1 -= wb.y;
      y0 = g.biasvolt * wb.x; y1 = g.biasvolt * wb.y;
    }
    nws[m] = pack2(n0, n1);
    ys[m] = pack2(y0, y1);
    wfin[2 * m] = 0.f - n0; wfin[2 * m + 1] = 0.f - n1;
    yfin[2 * m] = y0; yfin[2 * m + 1] = y1;
    live[2 * m] = live[2 * m + 1] = -1;
  }
  float xprev = g.has_bias ? g.biasvolt : 0.f;

  const float* wl = w + (FULL ? jbase + 2 * lane : 0);

  int sticky = INT_MAX;   // INT_MIN while some live output of this lane must be tested exactly at the next step
  const float tolbase = walk_tolerance_base(g);
  int qlim = 0;           // bits of the largest q that still goes to the exact tests (see walk_tolerance_base)
  auto step = [&](const float x, const float xprev, const uint64_t (&wv)[JP]) {
    const uint64_t x2 = pack2(x, x);
    int q[2 * JP];
#pragma unroll
    for (int m = 0; m < JP; ++m) unpack2i(fma2(x2, nws[m], ys[m]), q[2 * m], q[2 * m + 1]);
    int qmin;
    if constexpr (JP == 1) qmin = imin3(q[0], q[1], sticky);
    else if constexpr (JP == 2) qmin = imin3(imin3(q[0], q[1], q[2]), q[3], sticky);
    else qmin = imin3(imin3(q[0], q[1], q[2]), imin3(q[3], q[4], q[5]), imin3(q[6], q[7], sticky));
    if (__builtin_expect(__any_sync(0xffffffffu, qmin <= qlim), 0)) {
      // rare path: the reference's own rounded comparisons for the live outputs (see walk_row)
      bool again = false;
#pragma unroll
      for (int m = 0; m < JP; ++m) {
        float n[2], y[2];
        unpack2(nws[m], n[0], n[1]);
        unpack2(ys[m], y[0], y[1]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          // usually one output of one lane is concerned: skip the other half with a warp-uniform test
          if (!__any_sync(0xffffffffu, (q[2 * m + h] <= qlim) | (sticky < 0))) continue;
          const float wsum = 0.f - n[h];   // not -n: an exactly cancelled sum must read +0 as in the scalar walk
          const bool lv = live[2 * m + h] != 0;
          const bool fire = lv & ratio_gt(y[h], wsum, xprev) & ratio_le(y[h], wsum, x);
          if (fire) {
            live[2 * m + h] = 0;   // spike lies in (previous input, x]: keep the sums aside ...
            wfin[2 * m + h] = wsum;
            yfin[2 * m + h] = y[h];
            n[h] = CUDART_INF_F;   // ... and park the running weight sum where q stays +inf
          }
          again |= lv & !fire & (q[2 * m + h] <= qlim);
        }
        nws[m] = pack2(n[0], n[1]);
      }
      sticky = again ? INT_MIN : INT_MAX;
    }
#pragma unroll
    for (int m = 0; m < JP; ++m) {
      nws[m] = sub2(nws[m], wv[m]);
      ys[m] = fma2(x2, wv[m], ys[m]);
    }
  };
  const unsigned lane_off = (unsigned)jl[0];   // element offset of this lane's first pair within a weight row
  auto load_pair = [&](const float* wrow, int m) -> uint64_t {
    return __ldg(reinterpret_cast<const unsigned long long*>(FULL ? wrow + 64 * m : wrow + jl[m]));
  };

  bool all_done = false;
  auto load_row = [&](unsigned eoff, uint64_t (&wv)[JP]) {
    if constexpr (WS) {
      asm("ld.shared.b64 %0, [%1];" : "=l"(wv[0]) : "r"(eoff * wmul + ws_lane));
    } else if constexpr (JP == 1) {
      // one pair per lane: a 32-bit element offset from the (uniform) weight base measured faster than a
      // 64-bit per-lane pointer plus the entry's offset
      wv[0] = __ldg(reinterpret_cast<const unsigned long long*>(
          reinterpret_cast<const char*>(w) + (size_t)(eoff + lane_off) * 4u));
    } else {
      const float* wrow = wl + eoff;
#pragma unroll
      for (int m = 0; m < JP; ++m) wv[m] = load_pair(wrow, m);
    }
  };
  auto check_done = [&]() {
    int any_live = 0;
#pragma unroll
    for (int m = 0; m < 2 * JP; ++m) any_live |= live[m];
    all_done = !__any_sync(0xffffffffu, any_live != 0);
  };
  static_assert(CH % 2 == 0, "entries are fetched two at a time");
  auto chunk = [&](auto fetch2, int k0) {
    float xs[CH];
    uint64_t wv[CH][JP];
#pragma unroll
    for (int u = 0; u < CH; u += 2) {
      const uint4 e2 = fetch2(k0 + u);
      xs[u] = __uint_as_float(e2.x);
      load_row(e2.y, wv[u]);
      xs[u + 1] = __uint_as_float(e2.z);
      load_row(e2.w, wv[u + 1]);
    }
    qlim = __float_as_int(tolbase * fmaxf(fabsf(xs[0]), fabsf(xs[CH - 1])));   // inputs ascend: |x| peaks at an end
#pragma unroll
    for (int u = 0; u < CH; ++u) step(xs[u], u == 0 ? xprev : xs[u > 0 ? u - 1 : 0], wv[u]);
    xprev = xs[CH - 1];
  };
  auto single = [&](const WalkEntry e) {
    uint64_t wv[JP];
    if constexpr (WS) {
      load_row(e.y, wv);
    } else {
      const float* wrow = wl + e.y;
#pragma unroll
      for (int m = 0; m < JP; ++m) wv[m] = load_pair(wrow, m);
    }
    qlim = __float_as_int(tolbase * fabsf(__uint_as_float(e.x)));
    step(__uint_as_float(e.x), xprev, wv);
    xprev = __uint_as_float(e.x);
  };
  if constexpr (STAGE) {   // the list through shared memory, 32 entries at a time, read a block ahead (see walk_row)
    WalkEntry pre = make_uint2(0u, 0u);
    if (lane < nvalid) pre = __ldcg(ents + lane);
    int b = 0;
    for (int base = 0; base < nvalid && !all_done; base += 32, b ^= 32) {
      sbuf[b + lane] = pre;
      __syncwarp();
      if (base + 32 + lane < nvalid) pre = __ldcg(ents + base + 32 + lane);
      const int nb = min(32, nvalid - base);
      const WalkEntry* cur = sbuf + b;
      auto fetch2 = [&](int i) { return *reinterpret_cast<const uint4*>(cur + i); };
      int kk = 0;
#pragma unroll 1
      for (; kk + CH <= nb; kk += CH) chunk(fetch2, kk);
      for (; kk < nb; ++kk) single(cur[kk]);
      check_done();   // one "has every output fired" vote per block
    }
  } else {
    int k = 0;
    for (; k + CH <= nvalid && !all_done; k += CH) {
      // list entries bypass L1: it is kept for the weights
      chunk([&](int i) { return __ldcg(reinterpret_cast<const uint4*>(ents + i)); }, k);
      check_done();
    }
    if (!all_done)
      for (; k < nvalid; ++k) single(__ldcg(ents + k));
  }

#pragma unroll
  for (int m = 0; m < JP; ++m) {
    float n[2], y[2];
    unpack2(nws[m], n[0], n[1]);
    unpack2(ys[m], y[0], y[1]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // an output that stopped has fired; one that consumed every input fires iff it is armed
      bool fired = true;
      float ws = wfin[2 * m + h], yy = yfin[2 * m + h];
      if (live[2 * m + h]) {
        ws = 0.f - n[h]; yy = y[h];
        fired = ratio_gt(yy, ws, xprev);
      }
      float yv = g.maxv, iv = 0.f;
      if (fired) {
        iv = __fdividef(1.0f, ws);
        yv = yy * iv;
        if (yv >= g.maxv) { yv = g.maxv; iv = 0.f; }
      }
      if (jok[m]) {
        const int j = jbase + 2 * lane + 64 * m + h;
        y_row[j] = yv;
        if (inv_row != nullptr) inv_row[j] = iv;
        if (g.khist != nullptr) atomicAdd(g.khist + (yv < g.maxv ? entries_below(ents, nvalid, yv) : g.I + 1), 1);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- gather
// Where element i = lane + 32*n of a conv row sits in the receptive field, kept incrementally so that
// the per-element work has no integer division (the lane -> (kh, kw, c) map is the same for every row).
struct TapCursor {
  int kh, kw, c;
  __device__ __forceinline__ void init(const Geometry& g, int lane) {
    const int tap = lane / g.C;
    c = lane - tap * g.C;
    kh = tap / g.Kw;
    kw = tap - kh * g.Kw;
  }
  __device__ __forceinline__ void advance32(const Geometry& g) {
    c += 32;
    while (c >= g.C) {
      c -= g.C;
      if (++kw == g.Kw) { kw = 0; ++kh; }
    }
  }
};

// Loads one row, drops inputs above MAX-0.1, writes packed keys to dst[0..n) in index order and
// (if hist != nullptr) counts the four 8-bit digits of every kept key. Returns n. One warp.
// `start` is the cursor of element `lane` (conv only).
__device__ __forceinline__ int gather_row(const Geometry& g, const float* __restrict__ x, int r, int lane,
                                          u64* __restrict__ dst, unsigned* __restrict__ hist, const TapCursor& start) {
  const int I = g.I;
  const float maxcomp = g.maxv - 0.1f;
  int n = 0;
  int h0 = 0, w0 = 0;
  const float* xr = x + (size_t)r * I;
  TapCursor cur = start;
  if (g.is_conv) {
    const int nw = r % g.Nw;
    const int t = r / g.Nw;
    const int nh = t % g.Nh;
    const int b = t / g.Nh;
    h0 = nh * g.Sh - g.pad_top;
    w0 = nw * g.Sw - g.pad_left;
    xr = x + (size_t)b * g.H * g.W * g.C;
  }
  // four loads in flight per lane before anything depends on them: the loop is otherwise one global
  // load latency per 32 elements
  constexpr int kBatch = 4;
  for (int i0 = 0; i0 < I; i0 += 32 * kBatch) {
    float v[kBatch];
#pragma unroll
    for (int q = 0; q < kBatch; ++q) {
      const int i = i0 + 32 * q + lane;
      v[q] = g.maxv;
      if (i < I) {
        if (!g.is_conv) {
          v[q] = __ldg(xr + i);
        } else {
          const int h = h0 + cur.kh, ww = w0 + cur.kw;
          if (h >= 0 && h < g.H && ww >= 0 && ww < g.W) v[q] = __ldg(xr + ((size_t)h * g.W + ww) * g.C + cur.c);
        }
      }
      if (g.is_conv) cur.advance32(g);
    }
#pragma unroll
    for (int q = 0; q < kBatch; ++q) {
      const int i = i0 + 32 * q + lane;
      const bool keep = (i < I) && !(v[q] > maxcomp);
      const unsigned mask = __ballot_sync(0xffffffffu, keep);
      if (keep) {
        const uint32_t key = float_to_sortable(v[q]);
        dst[n + __popc(mask & ((1u << lane) - 1u))] = ((u64)key << 32) | (uint32_t)i;
        if (hist) {
          atomicAdd(&hist[key & 255u], 1u);
          atomicAdd(&hist[256 + ((key >> 8) & 255u)], 1u);
          atomicAdd(&hist[512 + ((key >> 16) & 255u)], 1u);
          atomicAdd(&hist[768 + (key >> 24)], 1u);
        }
      }
      n += __popc(mask);
    }
  }
  return n;
}

// ------------------------------------------------------------------------------------------- sorts
// In-place bitonic network for rows too long for two buffers; all threads of the CTA, one row.
// Every compare-exchange moves the smaller key to the lower index, so the virtual +inf elements at
// positions >= n never move and need no storage.
__device__ __forceinline__ void bitonic_sort_cta(u64* keys, int n, int tid) {
  int npad = 2;
  while (npad < n) npad <<= 1;
  const int half = npad >> 1;
  for (int k = 2; k <= npad; k <<= 1) {
    const int hk = k >> 1;
    for (int q = tid; q < half; q += kFwdThreads) {
      const int o = q & (hk - 1);
      const int base = (q - o) << 1;
      const int i = base + o, p = base + k - 1 - o;
      if (p < n) { const u64 va = keys[i], vb = keys[p]; if (va > vb) { keys[i] = vb; keys[p] = va; } }
    }
    __syncthreads();
    for (int j = hk >> 1; j >= 1; j >>= 1) {
      for (int q = tid; q < half; q += kFwdThreads) {
        const int o = q & (j - 1);
        const int i = ((q - o) << 1) + o, p = i + j;
        if (p < n) { const u64 va = keys[i], vb = keys[p]; if (va > vb) { keys[i] = vb; keys[p] = va; } }
      }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------------- compact warp sort
// The warp sort of snn_sort_kernel keeps keys (32-bit sortable value bits) and source indices (16 bit)
// in separate arrays and packs the four digit histograms two to a word: 12 bytes per input and 2 KB per
// warp instead of 16 bytes and 4 KB, which lets a third CTA (24 instead of 16 rows) be resident per SM
// at fan-in 577 -- the kernel is bound by shared-memory latency, so resident rows are what it needs.
struct SortBuffers {
  uint32_t* key;         // buffer b at key + b*I
  unsigned short* idx;   // buffer b at idx + b*I
  unsigned* hist;        // [0,256): digit 0 in bits 0..15, digit 1 in bits 16..31; [256,512): digits 2 and 3
  int I;
  // (the two buffers are addressed by offset, not through an array of pointers: a pointer picked at run time
  // out of an array loses its address space and every access through it becomes a generic load or store)
  __device__ __forceinline__ uint32_t* keys(int b) const { return key + b * I; }
  __device__ __forceinline__ unsigned short* idxs(int b) const { return idx + b * I; }
};
__host__ __device__ __forceinline__ size_t sort_bytes_per_warp(int I) {
  return (((size_t)12 * I + 15) & ~(size_t)15) + 2048;
}
__device__ __forceinline__ SortBuffers sort_buffers(unsigned char* base, int I) {
  SortBuffers b;
  b.key = reinterpret_cast<uint32_t*>(base);
  b.idx = reinterpret_cast<unsigned short*>(b.key + 2 * I);
  b.hist = reinterpret_cast<unsigned*>(base + (((size_t)12 * I + 15) & ~(size_t)15));
  b.I = I;
  return b;
}

// Where the taps of a conv row sit, relative to the row's top-left input pixel: built once per CTA, the same
// for every row. off[i] = ((kh*W + kw)*C + c) in elements, khw[i] = kh << 8 | kw (Kh, Kw <= 255). Both arrays
// are padded to a multiple of 128 entries so that a whole batch of loads may index them.
struct TapTable {
  const int* off;
  const unsigned short* khw;
};
__host__ __device__ __forceinline__ int tap_entries(int I) { return (I + 127) & ~127; }
__host__ __device__ __forceinline__ size_t tap_table_bytes(int I) { return (size_t)tap_entries(I) * 6; }

// Loads one row, drops inputs above MAX-0.1 and writes (sortable key, source index) of the rest to buffer 0
// in index order; returns their number and the smallest / largest key. One warp, no divergent branch: a tap
// outside the image (or past the end of the row) is a predicated-off load that reads as MAX and is dropped.
__device__ __forceinline__ int gather_row_compact(const Geometry& g, const float* __restrict__ x, int r, int lane,
                                                  const SortBuffers& sb, const TapTable& tt,
                                                  uint32_t& kmin, uint32_t& kmax) {
  const int I = g.I;
  const float maxcomp = g.maxv - 0.1f;
  int n = 0;
  int h0 = 0, w0 = 0;
  const float* xr = x + (size_t)r * I;
  if (g.is_conv) {
    const int nw = r % g.Nw;
    const int t = r / g.Nw;
    const int nh = t % g.Nh;
    const int b = t / g.Nh;
    h0 = nh * g.Sh - g.pad_top;
    w0 = nw * g.Sw - g.pad_left;
    // the row's top-left input pixel; may lie outside the image, in which case it is never dereferenced
    xr = x + ((ptrdiff_t)b * g.H * g.W + (ptrdiff_t)h0 * g.W + w0) * g.C;
  }
  uint32_t lmin = 0xFFFFFFFFu, lmax = 0u;
  const unsigned lt = (1u << lane) - 1u;
  constexpr int kBatch = 4;   // loads in flight per lane before anything depends on them
  for (int i0 = 0; i0 < I; i0 += 32 * kBatch) {
    float v[kBatch];
#pragma unroll
    for (int q = 0; q < kBatch; ++q) {
      const int i = i0 + 32 * q + lane;
      bool ok = i < I;
      ptrdiff_t o = i;
      if (g.is_conv) {
        const unsigned khw = tt.khw[i];
        o = tt.off[i];
        ok = ok && (unsigned)(h0 + (int)(khw >> 8)) < (unsigned)g.H && (unsigned)(w0 + (int)(khw & 255u)) < (unsigned)g.W;
      }
      v[q] = g.maxv;
      if (ok) v[q] = __ldg(xr + o);
    }
#pragma unroll
    for (int q = 0; q < kBatch; ++q) {
      const int i = i0 + 32 * q + lane;
      const bool keep = !(v[q] > maxcomp);   // a predicated-off load holds MAX
      const unsigned mask = __ballot_sync(0xffffffffu, keep);
      if (keep) {
        const uint32_t key = float_to_sortable(v[q]);
        const int pos = n + __popc(mask & lt);
        sb.key[pos] = key;
        sb.idx[pos] = (unsigned short)i;
        lmin = min(lmin, key);
        lmax = max(lmax, key);
      }
      n += __popc(mask);
    }
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    lmin = min(lmin, __shfl_xor_sync(0xffffffffu, lmin, d));
    lmax = max(lmax, __shfl_xor_sync(0xffffffffu, lmax, d));
  }
  kmin = lmin;
  kmax = lmax;
  return n;
}

// Rebase the keys of buffer 0 to key - kmin (order is kept, and the digits above the range of the row become
// zero, so their passes are not needed at all) and count the lowest `passes` 8-bit digits. One warp.
__device__ __forceinline__ void rebase_and_count(const SortBuffers& sb, int n, int lane, uint32_t kmin, int passes) {
  for (int i0 = 0; i0 < n; i0 += 128) {
    uint32_t k[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = i0 + 32 * q + lane;
      k[q] = i < n ? sb.key[i] - kmin : 0u;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = i0 + 32 * q + lane;
      if (i < n) {
        sb.key[i] = k[q];
        atomicAdd(&sb.hist[k[q] & 255u], 1u);
        if (passes > 1) atomicAdd(&sb.hist[(k[q] >> 8) & 255u], 1u << 16);
        if (passes > 2) atomicAdd(&sb.hist[256 + ((k[q] >> 16) & 255u)], 1u);
        if (passes > 3) atomicAdd(&sb.hist[256 + (k[q] >> 24)], 1u << 16);
      }
    }
  }
}

// n <= 32: rank every (key, index) against the others with shuffles. buffers 0 -> 1, one warp.
__device__ __forceinline__ void sort_small_compact(const SortBuffers& sb, int n, int lane) {
  const u64 e = lane < n ? (((u64)sb.key[lane] << 32) | sb.idx[lane]) : ~0ull;
  int rank = 0;
  for (int j = 0; j < n; ++j) {
    const u64 o = __shfl_sync(0xffffffffu, e, j);
    rank += o < e;
  }
  if (lane < n) { sb.keys(1)[rank] = (uint32_t)(e >> 32); sb.idxs(1)[rank] = (unsigned short)e; }
}

// Lanes of the warp whose 8-bit digit equals this lane's: eight ballots, one per bit (lanes without a key carry
// a digit >= 256 that is unique to them and are masked out by `actmask`). The match instruction gives the
// same mask in one go but runs on the SM's single address-divergence unit (about 55 cycles each), which bounds
// the kernel when every batch uses it; the ballots cost some 40 ALU instructions on the issuing scheduler's own
// pipe. The sort alternates between the two so that neither unit is the bottleneck.
__device__ __forceinline__ unsigned digit_peers(unsigned d, unsigned actmask) {
  unsigned same1 = actmask, any0 = 0u;   // AND of the ballots of this lane's set bits, OR of those of its clear bits
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const bool bit = (d >> b) & 1u;
    const unsigned m = __ballot_sync(0xffffffffu, bit);
    if (bit) same1 &= m; else any0 |= m;
  }
  return same1 & ~any0;
}

// Stable LSD radix sort, 8 bits per pass, one warp; returns which buffer (0/1) holds the result.
// `top_bits` = significant bits of the last digit (the keys are rebased, so the last digit of a row whose values
// span a few binades holds one or two bits): with at most two, that pass is a stable four-way split by two
// ballots per batch, with the class bases read from the digit's histogram -- no ranking, no histogram updates.
__device__ __forceinline__ int radix_sort_row_compact(const SortBuffers& sb, int n, int lane, int passes, int top_bits) {
  int cur = 0;
  const unsigned lt = (1u << lane) - 1u;
#pragma unroll 1
  for (int p = 0; p < passes; ++p) {
    unsigned* h = sb.hist + ((p >> 1) << 8);
    const int fs = (p & 1) << 4;   // this digit's 16-bit field inside the packed word
    if (p == passes - 1 && top_bits <= 2) {
      const unsigned c0 = (h[0] >> fs) & 0xFFFFu, c1 = (h[1] >> fs) & 0xFFFFu, c2 = (h[2] >> fs) & 0xFFFFu;
      if (c0 == (unsigned)n) continue;   // (cannot happen for a rebased top digit with range > 0; kept for safety)
      unsigned pos0 = 0u, pos1 = c0, pos2 = c0 + c1, pos3 = c0 + c1 + c2;   // next free slot of each class
      const uint32_t* srcK = sb.keys(cur);
      const unsigned short* srcI = sb.idxs(cur);
      uint32_t* dstK = sb.keys(cur ^ 1);
      unsigned short* dstI = sb.idxs(cur ^ 1);
      const int shift = 8 * p;
      for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        const bool act = i < n;
        const uint32_t k = act ? srcK[i] : 0u;
        const unsigned short ix = act ? srcI[i] : (unsigned short)0;
        const unsigned cls = (k >> shift) & 3u;
        const unsigned am = __ballot_sync(0xffffffffu, act);
        const unsigned b0 = __ballot_sync(0xffffffffu, act && (cls & 1u));
        const unsigned b1 = __ballot_sync(0xffffffffu, act && (cls & 2u));
        const unsigned m0 = am & ~b0 & ~b1, m1 = b0 & ~b1, m2 = b1 & ~b0, m3 = b0 & b1;
        const unsigned mine = cls == 0u ? m0 : (cls == 1u ? m1 : (cls == 2u ? m2 : m3));
        const unsigned at = cls == 0u ? pos0 : (cls == 1u ? pos1 : (cls == 2u ? pos2 : pos3));
        if (act) {
          const unsigned pos = at + __popc(mine & lt);
          dstK[pos] = k;
          dstI[pos] = ix;
        }
        pos0 += __popc(m0); pos1 += __popc(m1); pos2 += __popc(m2); pos3 += __popc(m3);
      }
      __syncwarp();
      cur ^= 1;
      continue;
    }
    unsigned wds[8], c[8], s = 0;
    bool single = false;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      wds[q] = h[lane * 8 + q];
      c[q] = (wds[q] >> fs) & 0xFFFFu;
      single |= (c[q] == (unsigned)n);
      s += c[q];
    }
    if (__any_sync(0xffffffffu, single)) continue;   // every key has the same digit here: nothing to do
    unsigned incl = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    unsigned run = incl - s;
#pragma unroll
    for (int q = 0; q < 8; ++q) {   // the field now holds the bin's running offset (<= n < 65536)
      h[lane * 8 + q] = (wds[q] & ~(0xFFFFu << fs)) | (run << fs);
      run += c[q];
    }
    __syncwarp();
    const uint32_t* srcK = sb.keys(cur);
    const unsigned short* srcI = sb.idxs(cur);
    uint32_t* dstK = sb.keys(cur ^ 1);
    unsigned short* dstI = sb.idxs(cur ^ 1);
    const int shift = 8 * p;
    constexpr int kSB = 4;   // batches of 32 keys whose loads and digit matches go ahead of the serial part
    for (int i0 = 0; i0 < n; i0 += 32 * kSB) {
      uint32_t k[kSB];
      unsigned short ix[kSB];
      unsigned d[kSB], peers[kSB];
      bool act[kSB];
#pragma unroll
      for (int q = 0; q < kSB; ++q) {
        const int i = i0 + 32 * q + lane;
        act[q] = i < n;
        k[q] = act[q] ? srcK[i] : 0u;
        ix[q] = act[q] ? srcI[i] : (unsigned short)0;
        d[q] = act[q] ? (k[q] >> shift) & 255u : 256u + (unsigned)lane;
      }
#pragma unroll
      for (int q = 0; q < kSB; ++q)
        peers[q] = (q & 1) ? digit_peers(d[q], __ballot_sync(0xffffffffu, act[q])) : __match_any_sync(0xffffffffu, d[q]);
#pragma unroll
      for (int q = 0; q < kSB; ++q) {
        // (a batch past the end of the row has no active lane and does nothing here: no branch around the
        // warp barriers, so that the compiler sees them in converged code)
        const unsigned before = peers[q] & lt;
        unsigned word = 0;
        if (act[q]) word = h[d[q]];
        __syncwarp();
        if (act[q] && before == 0) h[d[q]] = word + ((unsigned)__popc(peers[q]) << fs);
        __syncwarp();
        if (act[q]) {
          const unsigned pos = ((word >> fs) & 0xFFFFu) + __popc(before);
          dstK[pos] = k[q];
          dstI[pos] = ix[q];
        }
      }
    }
    __syncwarp();
    cur ^= 1;
  }
  return cur;
}

// ------------------------------------------------------------------------------------------- kernels
// Sort kernel: one warp per row. Shared memory per warp: two key buffers of I entries and the four
// digit histograms. Sorted keys go to keys_g[r*istride ..], their count to nvalid_g[r].
__global__ void __launch_bounds__(kFwdThreads)
snn_sort_kernel(const Geometry g, const float* __restrict__ x, WalkEntry* __restrict__ keys_g, int* __restrict__ nvalid_g,
                int istride, int row_begin, int row_end) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int I = g.I;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
  // conv: the tap table of the CTA comes first, then the warps' buffers
  TapTable tt = {nullptr, nullptr};
  unsigned char* warp_base = smem_raw;
  if (g.is_conv) {
    int* off = reinterpret_cast<int*>(smem_raw);
    unsigned short* khw = reinterpret_cast<unsigned short*>(off + tap_entries(I));
    for (int i = threadIdx.x; i < tap_entries(I); i += blockDim.x) {
      int o = 0;
      unsigned kk = 0;
      if (i < I) {
        const int tap = i / g.C, c = i - tap * g.C;
        const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
        o = (kh * g.W + kw) * g.C + c;
        kk = (unsigned)(kh << 8 | kw);
      }
      off[i] = o;
      khw[i] = (unsigned short)kk;
    }
    tt.off = off;
    tt.khw = khw;
    warp_base += (tap_table_bytes(I) + 15) & ~(size_t)15;
    __syncthreads();
  }
  const SortBuffers sb = sort_buffers(warp_base + (size_t)warp * sort_bytes_per_warp(I), I);
  for (int r = row_begin + blockIdx.x * wpc + warp; r < row_end; r += gridDim.x * wpc) {
    uint32_t kmin, kmax;
    const int n = gather_row_compact(g, x, r, lane, sb, tt, kmin, kmax);
    __syncwarp();
    int res = 0;
    uint32_t base = 0u;   // added back to the keys on the way out
    if (n > 32) {
      const uint32_t range = kmax - kmin;
      const int bits = 32 - __clz(range | 1u);
      const int passes = (bits + 7) >> 3;   // 8-bit digits that cover the range (1 when range < 256)
      const int top_bits = bits - 8 * (passes - 1);
      if (range != 0u) {
        for (int q = lane; q < 512; q += 32) sb.hist[q] = 0u;
        __syncwarp();
        rebase_and_count(sb, n, lane, kmin, passes);
        __syncwarp();
        res = radix_sort_row_compact(sb, n, lane, passes, top_bits);
        base = kmin;
      }   // else: every key is the same, index order is the sorted order
    } else {
      sort_small_compact(sb, n, lane);
      res = 1;
    }
    __syncwarp();
    WalkEntry* dst = keys_g + (size_t)r * istride;
    const uint32_t* rk = sb.keys(res);
    const unsigned short* ri = sb.idxs(res);
    for (int i = lane; i < n; i += 32)
      dst[i] = make_uint2(__float_as_uint(sortable_to_float(rk[i] + base)), (uint32_t)ri[i] * (uint32_t)g.J);
    if (lane == 0) nvalid_g[r] = n;
    __syncwarp();
  }
}

// Rows too long for two buffers per warp: one row per CTA at a time, in-place bitonic network.
__global__ void __launch_bounds__(kFwdThreads)
snn_sort_long_kernel(const Geometry g, const float* __restrict__ x, WalkEntry* __restrict__ keys_g,
                     int* __restrict__ nvalid_g, int istride) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  u64* keys = reinterpret_cast<u64*>(smem_raw);
  __shared__ int s_n;
  const int tid = threadIdx.x;
  for (int r = blockIdx.x; r < g.R; r += gridDim.x) {
    if (tid < 32) {
      TapCursor start = {0, 0, 0};
      if (g.is_conv) start.init(g, tid);
      const int n = gather_row(g, x, r, tid, keys, nullptr, start);
      if (tid == 0) s_n = n;
    }
    __syncthreads();
    const int n = s_n;
    bitonic_sort_cta(keys, n, tid);
    WalkEntry* dst = keys_g + (size_t)r * istride;
    for (int i = tid; i < n; i += kFwdThreads) {
      const u64 e = keys[i];
      dst[i] = make_uint2(__float_as_uint(key_value(e)), (uint32_t)e * (uint32_t)g.J);
    }
    if (tid == 0) nvalid_g[r] = n;
    __syncthreads();
  }
}

// Walk kernel: every warp takes (row, block of 32*JPT outputs) items, adjacent warps share a row.
template <int JPT, bool VECW, bool STAGE>
__global__ void __launch_bounds__(kFwdThreads, JPT <= 4 ? 4 : 1)   // up to four outputs per lane: 64 registers, 32 warps per SM
snn_walk_kernel(const Geometry g, const WalkEntry* __restrict__ keys_g, const int* __restrict__ nvalid_g, int istride,
                const float* __restrict__ w, float* __restrict__ out, int row_begin, int row_end) {
  __shared__ __align__(16) WalkEntry stage[STAGE ? kFwdWarps * 64 : 1];   // two blocks of 32 list entries per warp
  WalkEntry* sbuf = stage + (STAGE ? (threadIdx.x >> 5) * 64 : 0);
  const int J = g.J, R = g.R;
  const int lane = threadIdx.x & 31;
  const int jchunks = (J + 32 * JPT - 1) / (32 * JPT);
  const bool full_j = (J % (32 * JPT)) == 0;
  float* __restrict__ y_out = out;
  float* __restrict__ inv_out = g.infer ? nullptr : out + (size_t)R * J;
  const long items = (long)(row_end - row_begin) * jchunks;
  const long wstride = (long)gridDim.x * kFwdWarps;
  constexpr int CH = JPT >= 8 ? 2 : (JPT >= 4 ? 4 : 8);
  for (long item = (long)blockIdx.x * kFwdWarps + uniform_warp_index(); item < items; item += wstride) {
    const int rl = (int)(item / jchunks), jc = (int)(item - (long)rl * jchunks);
    const int r = row_begin + rl;
    const WalkEntry* krow = keys_g + (size_t)r * istride;
    const int n = __shfl_sync(0xffffffffu, __ldg(nvalid_g + r), 0);
    if (full_j)
      walk_row<JPT, CH, true, VECW, STAGE>(g, krow, n, w, jc * 32 * JPT, lane, y_out + (size_t)r * J, (inv_out ? inv_out + (size_t)r * J : nullptr), sbuf);
    else
      walk_row<JPT, CH, false, VECW, STAGE>(g, krow, n, w, jc * 32 * JPT, lane, y_out + (size_t)r * J, (inv_out ? inv_out + (size_t)r * J : nullptr), sbuf);
    if (STAGE) __syncwarp();   // the next row's first block goes into the buffer this row may have read last
  }
}

// The same items with the outputs of a lane held in pairs (walk_row2): a warp covers 64*JP outputs.
template <int JP, bool STAGE>
__global__ void __launch_bounds__(kFwdThreads)
snn_walk2_kernel(const Geometry g, const WalkEntry* __restrict__ keys_g, const int* __restrict__ nvalid_g, int istride,
                 const float* __restrict__ w, float* __restrict__ out, int row_begin, int row_end) {
  __shared__ __align__(16) WalkEntry stage[STAGE ? kFwdWarps * 64 : 1];   // two blocks of 32 list entries per warp
  WalkEntry* sbuf = stage + (STAGE ? (threadIdx.x >> 5) * 64 : 0);
  const int J = g.J, R = g.R;
  const int lane = threadIdx.x & 31;
  const int jchunks = (J + 64 * JP - 1) / (64 * JP);
  const bool full_j = (J % (64 * JP)) == 0;
  float* __restrict__ y_out = out;
  float* __restrict__ inv_out = g.infer ? nullptr : out + (size_t)R * J;
  const long items = (long)(row_end - row_begin) * jchunks;
  const long wstride = (long)gridDim.x * kFwdWarps;
  for (long item = (long)blockIdx.x * kFwdWarps + uniform_warp_index(); item < items; item += wstride) {
    const int rl = (int)(item / jchunks), jc = (int)(item - (long)rl * jchunks);
    const int r = row_begin + rl;
    const WalkEntry* krow = keys_g + (size_t)r * istride;
    const int n = __shfl_sync(0xffffffffu, __ldg(nvalid_g + r), 0);
    if (full_j)
      walk_row2<JP, (JP >= 2 ? 4 : 8), true, STAGE>(g, krow, n, w, jc * 64 * JP, lane, y_out + (size_t)r * J, (inv_out ? inv_out + (size_t)r * J : nullptr), sbuf);
    else
      walk_row2<JP, (JP >= 2 ? 4 : 8), false, STAGE>(g, krow, n, w, jc * 64 * JP, lane, y_out + (size_t)r * J, (inv_out ? inv_out + (size_t)r * J : nullptr), sbuf);
    if (STAGE) __syncwarp();
  }
}

// ---- the pairs walk with its weights staged in shared memory ---------------------------------------------
// Where all fan-in rows of 64 outputs fit into one CTA's shared memory ((I + bias) * 256 bytes: up to about 800
// rows), a persistent CTA of 32 warps copies that slice of the weight matrix in once -- one asynchronous bulk copy
// (cp.async.bulk) per weight row, all completing on one mbarrier -- and every step of every walk then reads its
// weight pair with one shared-memory load instead of a global load through L1. CTA c takes output slice
// c % (J/64) and every (gridDim.x / (J/64))-th row of that slice.
constexpr int kSmemwThreads = 1024;
constexpr int kSmemwWarps = kSmemwThreads / 32;
constexpr long long kSmemwWaitClocks = 2000000000LL;   // SM clocks a CTA waits for its weight copies (about a second)
__device__ unsigned g_walk_copy_timeouts = 0u;          // CTAs that gave up waiting since the library was loaded

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

template <bool STAGE>
__global__ void __launch_bounds__(kSmemwThreads, 1)
snn_walk2_smemw_kernel(const Geometry g, const WalkEntry* __restrict__ keys_g, const int* __restrict__ nvalid_g,
                       int istride, const float* __restrict__ w, float* __restrict__ out, int row_begin, int row_end,
                       unsigned wmul) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long copy_done;
  const int J = g.J, R = g.R;
  const int rows_w = g.I + g.has_bias;
  float* ws = reinterpret_cast<float*>(smem_raw);                                        // [rows_w][64]
  WalkEntry* stage = reinterpret_cast<WalkEntry*>(smem_raw + (size_t)rows_w * 256);      // [32 warps][64 entries]
  const int lane = threadIdx.x & 31;
  const int warp = uniform_warp_index();
  const int slices = J >> 6;
  const int slice = blockIdx.x % slices;
  const int j0 = slice << 6;
  const unsigned bar = smem_u32(&copy_done);

  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((unsigned)rows_w * 256u) : "memory");
    __syncwarp();
    for (int row = lane; row < rows_w; row += 32)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 256, [%2];"
                   ::"r"(smem_u32(ws + row * 64)), "l"(__cvta_generic_to_global(w + (size_t)row * J + j0)), "r"(bar) : "memory");
  }
  // Every thread waits for the copies itself (phase 0 of the barrier), for at most about a second of SM clocks. If
  // they have not arrived by then the CTA counts a timeout and walks with the weights read from global memory, like
  // snn_walk2_kernel; before it leaves it gives the copies the same time once more, so that none is in flight into
  // shared memory that the next CTA on this SM owns.
  auto copies_arrived = [&]() {
    const long long t0 = clock64();
    bool arrived = false;
    while (!arrived && clock64() - t0 < kSmemwWaitClocks) {
      unsigned ok;
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(ok) : "r"(bar) : "memory");
      arrived = ok != 0u;
    }
    return arrived;
  };
  const bool staged = !__syncthreads_or(!copies_arrived());
  if (!staged && threadIdx.x == 0) atomicAdd(&g_walk_copy_timeouts, 1u);

  WalkEntry* sbuf = stage + warp * 64;
  float* __restrict__ y_out = out;
  float* __restrict__ inv_out = g.infer ? nullptr : out + (size_t)R * J;
  const unsigned ws_lane = smem_u32(ws) + 8u * (unsigned)lane;
  const int ctas = gridDim.x / slices;                 // CTAs that share this slice (the host makes gridDim.x a multiple)
  const int cta = blockIdx.x / slices;
  for (long rl = (long)cta * kSmemwWarps + warp; rl < row_end - row_begin; rl += (long)ctas * kSmemwWarps) {
    const int r = row_begin + (int)rl;
    const WalkEntry* krow = keys_g + (size_t)r * istride;
    const int n = __shfl_sync(0xffffffffu, __ldg(nvalid_g + r), 0);
    float* yr = y_out + (size_t)r * J;
    float* ir = inv_out ? inv_out + (size_t)r * J : nullptr;
    if (staged) walk_row2<1, 8, true, STAGE, true>(g, krow, n, w, j0, lane, yr, ir, sbuf, ws_lane, wmul);
    else walk_row2<1, 8, true, STAGE, false>(g, krow, n, w, j0, lane, yr, ir, sbuf);
    if (STAGE) __syncwarp();
  }
  if (!staged) {
    __syncthreads();
    (void)copies_arrived();
  }
}

int key_stride(const Geometry& g) { return (g.I + 3) & ~3; }  // a multiple of four entries: rows of keys start 32-byte aligned

size_t keys_bytes(const Geometry& g) { return (size_t)g.R * key_stride(g) * sizeof(u64); }
// list lengths, then 256 bytes that hold the weight bound of the walk (one float)
size_t nvalid_only_bytes(const Geometry& g) { return ((size_t)g.R * sizeof(int) + 255) & ~(size_t)255; }
size_t nvalid_bytes(const Geometry& g) { return nvalid_only_bytes(g) + 256; }

template <int JPT, bool VECW>
int launch_walk(const Geometry& g, const WalkEntry* keys_g, const int* nvalid_g, const float* w, float* out,
                const LaunchInfo& li, cudaStream_t s, int row_begin, int row_end, bool stage) {
  const int jchunks = (g.J + 32 * JPT - 1) / (32 * JPT);
  const long items = (long)(row_end - row_begin) * jchunks;
  long grid = (items + kFwdWarps - 1) / kFwdWarps;
  const long cap = (long)li.num_sms * 8;
  if (grid > cap) grid = cap;
  if (stage) snn_walk_kernel<JPT, VECW, true><<<(int)grid, kFwdThreads, 0, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end);
  else snn_walk_kernel<JPT, VECW, false><<<(int)grid, kFwdThreads, 0, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

template <int JP>
int launch_walk2(const Geometry& g, const WalkEntry* keys_g, const int* nvalid_g, const float* w, float* out,
                 const LaunchInfo& li, cudaStream_t s, int row_begin, int row_end, bool stage) {
  const int jchunks = (g.J + 64 * JP - 1) / (64 * JP);
  const long items = (long)(row_end - row_begin) * jchunks;
  long grid = (items + kFwdWarps - 1) / kFwdWarps;
  const long cap = (long)li.num_sms * 8;
  if (grid > cap) grid = cap;
  if (stage) snn_walk2_kernel<JP, true><<<(int)grid, kFwdThreads, 0, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end);
  else snn_walk2_kernel<JP, false><<<(int)grid, kFwdThreads, 0, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

// The pairs walk with the weights staged in shared memory: fan-out a power-of-two multiple of 64, weights 16-byte
// aligned, all (I + bias) rows of a 64-output slice plus the list staging buffers within one CTA's shared memory.
bool walk_smemw_ok(const Geometry& g, const float* w, const LaunchInfo& li, size_t* smem_bytes, int* wmul) {
  if ((g.J != 64 && g.J != 128 && g.J != 256) || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return false;
  const size_t rows_w = (size_t)g.I + g.has_bias;
  const size_t smem = rows_w * 256 + (size_t)kSmemwWarps * 64 * sizeof(WalkEntry);
  if (smem + 2048 > (size_t)li.max_smem_optin || rows_w * 256 >= (1u << 20)) return false;
  if ((g.J >> 6) > li.num_sms) return false;
  *smem_bytes = smem;
  *wmul = 256 / g.J;
  return true;
}

int launch_walk2_smemw(const Geometry& g, const WalkEntry* keys_g, const int* nvalid_g, const float* w, float* out,
                       const LaunchInfo& li, cudaStream_t s, int row_begin, int row_end, bool stage, size_t smem,
                       int wmul) {
  const int slices = g.J >> 6;
  const long rows = row_end - row_begin;
  long per_slice = li.num_sms / slices;                       // persistent: one CTA per SM
  const long need = (rows + kSmemwWarps - 1) / kSmemwWarps;
  if (per_slice > need) per_slice = need;
  if (per_slice < 1) per_slice = 1;
  const int grid = (int)(per_slice * slices);
  if (stage) {
    if (cudaFuncSetAttribute(snn_walk2_smemw_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return E_CUDA;
    snn_walk2_smemw_kernel<true><<<grid, kSmemwThreads, smem, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end, (unsigned)wmul);
  } else {
    if (cudaFuncSetAttribute(snn_walk2_smemw_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return E_CUDA;
    snn_walk2_smemw_kernel<false><<<grid, kSmemwThreads, smem, s>>>(g, keys_g, nvalid_g, key_stride(g), w, out, row_begin, row_end, (unsigned)wmul);
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

// Lists of a conv layer are built by per-pixel sorting and merging when the geometry allows it and the row
// sort would sort every input pixel several times over (3x3 stride 1: nine times).
bool use_merge_lists(const Geometry& g, const Options& opt) {
  const int want = opt.list_builder & 3;
  if (want == 1 || want == 3 || !merge_lists_supported(g)) return false;
  return true;
}

// Short rows (a first layer on a few image channels) are sorted by a network in registers.
bool use_small_rows(const Geometry& g, const Options& opt) {
  const int want = opt.list_builder & 3;
  if (want == 1 || want == 2 || !small_rows_supported(g)) return false;
  return true;
}

}  // namespace

unsigned long long walk_copy_timeouts() {
  unsigned n = 0;
  if (cudaMemcpyFromSymbol(&n, g_walk_copy_timeouts, sizeof(n)) != cudaSuccess) note_cuda_error(cudaGetLastError());
  return n;
}

size_t forward_workspace_bytes(const Geometry& g) {
  // sorted lists, their lengths, and (conv layers that qualify) the scratch of the merging list builder
  return keys_bytes(g) + nvalid_bytes(g) + (merge_lists_shape_ok(g) ? merge_lists_bytes(g) : 0);
}

int launch_forward(const Geometry& g_in, const float* x, const float* w, float* out, void* ws, size_t ws_bytes,
                   const LaunchInfo& li, const Options& opt, cudaStream_t s) {
  if (!ws || ws_bytes < forward_workspace_bytes(g_in)) return E_WORKSPACE;
  WalkEntry* keys_g = static_cast<WalkEntry*>(ws);
  int* nvalid_g = reinterpret_cast<int*>(static_cast<unsigned char*>(ws) + keys_bytes(g_in));
  float* wbound = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + keys_bytes(g_in) + nvalid_only_bytes(g_in));
  void* merge_scratch = static_cast<unsigned char*>(ws) + keys_bytes(g_in) + nvalid_bytes(g_in);
  Geometry g = g_in;
  g.wbound = wbound;
  const int istride = key_stride(g);

  const int fparts = opt.forward_parts;
  if (fparts & 2) {   // the walk's bound on the weight sums (see walk_tolerance_base)
    const int rows_w = g.I + g.has_bias;
    int per = (rows_w + kBoundMaxCtas - 1) / kBoundMaxCtas;
    per = (per + 7) & ~7;                                // whole rounds of the CTA's eight warps
    g.wbound_n = (rows_w + per - 1) / per;
    snn_wbound_kernel<<<g.wbound_n, 256, 0, s>>>(w, rows_w, g.J, per, wbound);
    count_launch();
    if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  }
  // Outputs per lane: more of them amortise the per-step cost (list entry, address, vote) over more
  // outputs, fewer give more (row, output block) items to spread over the SMs. `cost` is the measured number
  // of instructions per warp-step, `ctas` how many CTAs fit per SM; with few items pick the smallest
  // estimate of (waves of items) x (cost of a step).
  auto pick = [&](int unit, const double (&cost)[4], const int (&ctas)[4], int top) {
    int best_c = top;
    const double items_top = (double)g.R * ((g.J + unit * (1 << top) - 1) / (unit * (1 << top)));
    if (items_top < 4.0 * li.num_sms * ctas[top] * kFwdWarps) {
      double best = 0;
      for (int c = 0; c <= top; ++c) {
        const int per = unit * (1 << c);
        const double items = (double)g.R * ((g.J + per - 1) / per);
        const double slots = (double)li.num_sms * ctas[c] * kFwdWarps;
        const double est = (double)(long)(items / slots + 0.999) * cost[c];
        if (c == 0 || est < best) { best = est; best_c = c; }
      }
    }
    return best_c;
  };
  // Variants of the walk: 1 = output pairs in 64-bit registers, 64 outputs per warp (fan-out <= 64, or few rows:
  // more warps); 3 = scalar, 2, 4 or 8 consecutive outputs per lane read by 8/16-byte loads (fan-out > 64);
  // 2 = scalar with outputs lane + 32*m (odd fan-out or unaligned weights).
  const bool al8 = (g.J % 2 == 0) && (reinterpret_cast<uintptr_t>(w) % 8 == 0);
  const bool al16 = (g.J % 4 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  const bool al32 = al16 && (g.J % 8 == 0);
  const double cost[4] = {19.0, 24.0, 39.0, 62.0};
  const int ctas[4] = {6, 4, 4, 2};
  // (eight outputs per lane exist as a variant but were measured slower than four on every layer of the benchmark
  // networks -- 1.91 against 1.32 ms on the 2305 x 256 layer: 98 registers, two CTAs per SM -- and are never picked)
  int jsel = pick(32, cost, ctas, g.J <= 32 ? 0 : (g.J <= 64 ? 1 : 2));
  int variant = 2;
  if (al8) variant = (g.J <= 64 || jsel < 2) ? 1 : 3;
  if ((opt.walk_layout & 3) != 0) {
    variant = opt.walk_layout & 3;
    if (variant != 2 && !al8) variant = 2;
  }
  const bool stage = (opt.walk_layout & 4) == 0;   // list entries through shared memory (4: straight from global memory)
  if (opt.walk_outputs != 0) jsel = opt.walk_outputs - 1;
  if (jsel == 3 && !(variant == 3 && al32)) jsel = 2;   // eight outputs per lane exist only as consecutive outputs
  if (variant == 3 && jsel == 2 && !al16) jsel = 1;
  size_t smemw_bytes = 0;
  int smemw_shift = 0;
  // weights staged in shared memory: where they fit, for fan-out 64 with enough rows to keep one CTA of 32 warps
  // per SM busy (measured 13-16 % faster than the global-memory pairs walk; at fan-out 128 four outputs per lane
  // from global memory are 5 % faster than two staged slices); walk_layout 8 asks for it wherever it fits, a named
  // layout switches it off
  const bool smemw = walk_smemw_ok(g, w, li, &smemw_bytes, &smemw_shift) &&
                     ((opt.walk_layout & 8) != 0 || ((opt.walk_layout & 3) == 0 && g.J == 64 && g.R >= 8192));
  auto walk = [&](cudaStream_t st, int r0, int r1) -> int {
    if (!(fparts & 2)) return OK;
    if (smemw) return launch_walk2_smemw(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage, smemw_bytes, smemw_shift);
    if (variant == 1) {
      // pairs layout: 64 outputs per warp, or (walk_outputs 3) 128 as two pairs per lane
      if (jsel >= 2) return launch_walk2<2>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
      return launch_walk2<1>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
    }
    if (jsel == 0) return launch_walk<1, false>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
    if (variant == 3) {
      if (jsel == 1) return launch_walk<2, true>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
      if (jsel == 2) return launch_walk<4, true>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
      return launch_walk<8, true>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
    }
    if (jsel == 1) return launch_walk<2, false>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
    return launch_walk<4, false>(g, keys_g, nvalid_g, w, out, li, st, r0, r1, stage);
  };

  if (use_merge_lists(g, opt)) {
    if (fparts & 1) {
      const int rc = launch_merge_lists(g, x, keys_g, nvalid_g, istride, merge_scratch, (opt.list_builder >> 2) - 1, li, s);
      if (rc != OK) return rc;
    }
    return walk(s, 0, g.R);
  }
  if (use_small_rows(g, opt)) {
    if (fparts & 1) {
      const int rc = launch_small_rows(g, x, keys_g, nvalid_g, istride, li, s);
      if (rc != OK) return rc;
    }
    return walk(s, 0, g.R);
  }

  const size_t budget = (size_t)li.max_smem_optin - 1024;
  const size_t per_warp = sort_bytes_per_warp(g.I);
  const size_t table_min = g.is_conv ? ((tap_table_bytes(g.I) + 15) & ~(size_t)15) : 0;
  if (table_min + per_warp > budget || g.I > 65535 || (g.is_conv && (g.Kh > 255 || g.Kw > 255))) {
    // rows too long for the warp sort: one CTA-wide bitonic sort per row, then the walk
    const size_t smem = (size_t)g.I * sizeof(u64);
    if (smem > budget) return E_UNSUPPORTED;
    if (cudaFuncSetAttribute(snn_sort_long_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget) != cudaSuccess)
      return E_CUDA;
    int grid = g.R < li.num_sms ? g.R : li.num_sms;
    if (fparts & 1) {
      snn_sort_long_kernel<<<grid, kFwdThreads, smem, s>>>(g, x, keys_g, nvalid_g, istride);
      count_launch();
      if (cudaGetLastError() != cudaSuccess) return E_CUDA;
    }
    return walk(s, 0, g.R);
  }

  // warps per CTA and CTAs per SM: the combination that keeps the most rows (warps) resident per SM
  const size_t table = g.is_conv ? ((tap_table_bytes(g.I) + 15) & ~(size_t)15) : 0;
  int wpc = 1, ctas_per_sm = 1;
  {
    int best = 0;
    for (int cand = kFwdWarps; cand >= 1; --cand) {
      if (table + per_warp * cand > budget) continue;
      int c = (int)(((size_t)li.max_smem_optin) / (table + per_warp * cand + 1024));
      if (c > 4) c = 4;
      if (c < 1) c = 1;
      if (cand * c > best) { best = cand * c; wpc = cand; ctas_per_sm = c; }
    }
  }
  const size_t smem = table + per_warp * wpc;
  if (cudaFuncSetAttribute(snn_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget) != cudaSuccess)
    return E_CUDA;
  auto sort = [&](cudaStream_t st, int r0, int r1) -> int {
    long grid = ((long)(r1 - r0) + wpc - 1) / wpc;
    const long cap = (long)li.num_sms * ctas_per_sm;
    if (grid > cap) grid = cap;
    snn_sort_kernel<<<(int)grid, wpc * 32, smem, st>>>(g, x, keys_g, nvalid_g, istride, r0, r1);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
  };

  // Sort, then walk, on the caller's stream. (Running the next block's sort beside the current block's walk
  // on a second stream was measured and gains nothing: both kernels fill the SMs on their own.)
  int rc = (fparts & 1) ? sort(s, 0, g.R) : OK;
  if (rc != OK) return rc;
  return walk(s, 0, g.R);
}

}  // namespace snntc
