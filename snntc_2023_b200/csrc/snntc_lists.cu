// Sorted input lists of a stride-1 convolution (SnnCv, snntc/snncv_kernels.cu.cc:111-167: the reference
// materialises every receptive field with extract_image_patches and sorts each one with a segmented sort).
//
// Neighbouring receptive fields of a 3x3 stride-1 convolution share six of their nine input pixels, so sorting
// every field on its own sorts every input value nine times. Here every input value is sorted ONCE and the
// fields are assembled by merging:
//   1. pixel runs   one warp per input pixel: the pixel's C channel values, minus those that never spike
//                   (> MAX - 0.1, NaN), sorted by a bitonic network held in registers (shuffles between lanes);
//   2. row runs     one thread per (input row h, output column nw): sequential merge of the Kw pixel runs
//                   (h, nw - pad_left + kw) -- shared by the Kh receptive fields that contain that row segment;
//   3. field lists  one thread per receptive field: sequential merge of its Kh row runs, written in the format
//                   the walk kernels read: (x, element offset of weight row ((kh*Kw+kw)*C+c)).
// Where a layer has too few row segments or fields to fill the GPU with one thread each (deep layers: small
// images, many channels), 2 to 16 neighbouring threads share a merge, cut into pieces by value.
// A sequential two- or three-way merge costs a few dozen instructions per entry and thread and needs no
// cooperation between threads; the per-field radix sort it replaces spends about five hundred per entry.
// Each thread streams through its own runs, so what bounds these kernels is the number of memory transactions:
// the merges read and write 32 bytes (four entries) at a time.
// The order among equal input values differs from a per-field sort's; no output can spike between two equal
// inputs, so the walk's result does not depend on it.
#include "snntc_common.cuh"
#include "snntc_merge.cuh"

#include <math_constants.h>

namespace snntc {

namespace {

typedef unsigned long long u64;

constexpr int kListThreads = 128;
constexpr int kPixelWarps = 8;

// Bitonic sort of 32*EPL keys, EPL per lane: element e = lane*EPL + m lives in v[m] of lane e / EPL.
// Ascending; afterwards element e has rank e.
template <int EPL>
__device__ __forceinline__ void warp_bitonic_sort(u64 (&v)[EPL], int lane) {
#pragma unroll
  for (int k = 2; k <= 32 * EPL; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j >= 1; j >>= 1) {
      if (j >= EPL) {
        const int lj = j / EPL;                       // partner lane = lane ^ lj, same slot m
        const bool lower = (lane & lj) == 0;          // this lane holds the lower index of each pair
#pragma unroll
        for (int m = 0; m < EPL; ++m) {
          const u64 o = __shfl_xor_sync(0xffffffffu, v[m], lj);
          const bool asc = (((lane * EPL + m) & k) == 0) || (k == 32 * EPL);
          const bool take_min = (asc == lower);
          const bool o_less = o < v[m];
          v[m] = (take_min == o_less) ? o : v[m];
        }
      } else {
#pragma unroll
        for (int m = 0; m < EPL; ++m) {
          const int p = m ^ j;
          if (p > m) {
            const bool asc = (((lane * EPL + m) & k) == 0) || (k == 32 * EPL);
            const u64 a = v[m], b = v[p];
            const bool sw = asc ? (a > b) : (a < b);
            v[m] = sw ? b : a;
            v[p] = sw ? a : b;
          }
        }
      }
    }
  }
}

// Sort of 32*EPL keys for an EPL that is no power of two (the bitonic network above would round it up: 160 keys
// would be sorted as 256). Every lane sorts its own EPL keys; the lanes then run the bitonic network over their
// BLOCKS, a compare-exchange being a merge-split: against the partner's block in reverse, min(mine[i], theirs[EPL-1-i])
// over i are the EPL smallest keys of both blocks, the maxima the EPL largest; what a lane keeps is sorted again
// (odd-even transposition: EPL (EPL - 1) / 2 exchanges). Same result layout: element lane*EPL + m has rank lane*EPL + m.
template <int EPL>
__device__ __forceinline__ void lane_sort(u64 (&v)[EPL]) {
#pragma unroll
  for (int round = 0; round < EPL; ++round) {
#pragma unroll
    for (int i = round & 1; i + 1 < EPL; i += 2) {
      const u64 a = v[i], b = v[i + 1];
      const bool sw = a > b;
      v[i] = sw ? b : a;
      v[i + 1] = sw ? a : b;
    }
  }
}
template <int EPL>
__device__ __forceinline__ void warp_block_sort(u64 (&v)[EPL], int lane) {
  lane_sort<EPL>(v);
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j >= 1; j >>= 1) {
      const bool lower = (lane & j) == 0;
      const bool asc = (lane & k) == 0 || k == 32;
      const bool keep_low = asc == lower;
      u64 o[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) o[i] = __shfl_xor_sync(0xffffffffu, v[EPL - 1 - i], j);
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const bool o_less = o[i] < v[i];
        v[i] = (keep_low == o_less) ? o[i] : v[i];
      }
      lane_sort<EPL>(v);
    }
  }
}
template <int EPL>
__device__ __forceinline__ void warp_sort(u64 (&v)[EPL], int lane) {
  if constexpr ((EPL & (EPL - 1)) == 0) warp_bitonic_sort<EPL>(v, lane);
  else warp_block_sort<EPL>(v, lane);
}

// Sorts the n <= 32*EPL real keys of v (the other slots hold ~0) and writes them as a run. A pixel that has at most
// half its slots filled -- most pixels of a hidden layer: about half of a layer's inputs never spike -- is first
// compacted through `buf` (16*EPL keys of shared memory per warp) into half the slots, again and again if it can
// be, so that the network it goes through fits its real keys, not its channel count.
template <int EPL>
__device__ __forceinline__ void sort_and_write_run(u64 (&v)[EPL], int n, int lane, u64* __restrict__ buf,
                                                   WalkEntry* __restrict__ dst, int J) {
  if constexpr (EPL >= 2 && (EPL & 1) == 0) {
    if (n <= 16 * EPL) {   // warp-uniform
      const unsigned lt = (1u << lane) - 1u;
      int base = 0;
      __syncwarp();
#pragma unroll
      for (int m = 0; m < EPL; ++m) {
        const bool keep = v[m] != ~0ull;
        const unsigned mask = __ballot_sync(0xffffffffu, keep);
        if (keep) buf[base + __popc(mask & lt)] = v[m];
        base += __popc(mask);
      }
      __syncwarp();
      u64 w[EPL / 2];
#pragma unroll
      for (int m = 0; m < EPL / 2; ++m) w[m] = (m * 32 + lane < n) ? buf[m * 32 + lane] : ~0ull;
      sort_and_write_run<EPL / 2>(w, n, lane, buf, dst, J);
      return;
    }
  }
  warp_sort<EPL>(v, lane);
#pragma unroll
  for (int m = 0; m < EPL; ++m) {
    const int rank = lane * EPL + m;
    if (rank < n)
      dst[rank] = make_uint2(__float_as_uint(sortable_to_float((uint32_t)(v[m] >> 32))), (uint32_t)v[m] * (uint32_t)J);
  }
}

// One warp per input pixel p = (b*H + h)*W + w: runs[p*stride ..] receives the pixel's inputs that can spike
// as (float bits, c*J) in ascending order followed by a terminator; counts[p] their number.
template <int EPL>
__global__ void __launch_bounds__(kPixelWarps * 32)
snn_pixel_runs_kernel(const float* __restrict__ x, int npix, int C, int J, float maxcomp,
                      WalkEntry* __restrict__ runs, int* __restrict__ counts, int stride) {
  __shared__ u64 compact[kPixelWarps][EPL >= 2 ? 16 * EPL : 1];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int p = blockIdx.x * kPixelWarps + warp; p < npix; p += gridDim.x * kPixelWarps) {
    const float* xp = x + (size_t)p * C;
    u64 v[EPL];
    int n = 0;
#pragma unroll
    for (int m = 0; m < EPL; ++m) {
      const int c = m * 32 + lane;                    // coalesced: the network does not care where a key starts
      float val = CUDART_INF_F;
      if (c < C) val = __ldg(xp + c);
      const bool keep = val <= maxcomp;               // false for NaN and for inputs that never spike
      v[m] = keep ? (((u64)float_to_sortable(val) << 32) | (unsigned)c) : ~0ull;
      n += __popc(__ballot_sync(0xffffffffu, keep));
    }
    WalkEntry* dst = runs + (size_t)p * stride;
    sort_and_write_run<EPL>(v, n, lane, compact[warp], dst, J);
    if (lane == 0) {
      dst[n] = make_uint2(kRunEndBits, 0u);
      counts[p] = n;
    }
  }
}

// Rows of at most 256 inputs (the first layer of a network: a few channels under a small kernel), one warp per
// row: the inputs that can spike, gathered tap by tap through a table in shared memory, sorted by the same
// register network on (value, source index) -- ties in index order, like a stable sort -- and written straight
// as the list the walk reads. A dense row is its own table.
template <int EPL>
__global__ void __launch_bounds__(kPixelWarps * 32)
snn_small_rows_kernel(const Geometry g, const float* __restrict__ x, WalkEntry* __restrict__ lists,
                      int* __restrict__ nvalid, int istride) {
  __shared__ int tap_off[32 * EPL];
  __shared__ unsigned short tap_khw[32 * EPL];
  const int I = g.I;
  if (g.is_conv) {
    for (int i = threadIdx.x; i < 32 * EPL; i += blockDim.x) {
      int o = 0;
      unsigned kk = 0;
      if (i < I) {
        const int tap = i / g.C, c = i - tap * g.C;
        const int kh = tap / g.Kw, kw = tap - kh * g.Kw;
        o = (kh * g.W + kw) * g.C + c;
        kk = (unsigned)(kh << 8 | kw);
      }
      tap_off[i] = o;
      tap_khw[i] = (unsigned short)kk;
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float maxcomp = g.maxv - 0.1f;
  for (int r = blockIdx.x * kPixelWarps + warp; r < g.R; r += gridDim.x * kPixelWarps) {
    const float* xr = x + (size_t)r * I;
    int h0 = 0, w0 = 0;
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
    u64 v[EPL];
    int n = 0;
#pragma unroll
    for (int m = 0; m < EPL; ++m) {
      const int i = m * 32 + lane;
      bool ok = i < I;
      ptrdiff_t o = i;
      if (g.is_conv) {
        const unsigned khw = tap_khw[i];
        o = tap_off[i];
        ok = ok && (unsigned)(h0 + (int)(khw >> 8)) < (unsigned)g.H && (unsigned)(w0 + (int)(khw & 255u)) < (unsigned)g.W;
      }
      float val = CUDART_INF_F;
      if (ok) val = __ldg(xr + o);
      const bool keep = val <= maxcomp;               // false for NaN, padding and inputs that never spike
      v[m] = keep ? (((u64)float_to_sortable(val) << 32) | (unsigned)i) : ~0ull;
      n += __popc(__ballot_sync(0xffffffffu, keep));
    }
    warp_sort<EPL>(v, lane);
    WalkEntry* dst = lists + (size_t)r * istride;
#pragma unroll
    for (int m = 0; m < EPL; ++m) {
      const int rank = lane * EPL + m;
      if (rank < n)
        dst[rank] = make_uint2(__float_as_uint(sortable_to_float((uint32_t)(v[m] >> 32))),
                               (uint32_t)v[m] * (uint32_t)g.J);
    }
    if (lane == 0) nvalid[r] = n;
  }
}

__device__ __align__(32) const WalkEntry g_empty_run[4] = {{kRunEndBits, 0u}, {kRunEndBits, 0u}, {kRunEndBits, 0u}, {kRunEndBits, 0u}};

// How merge3_runs_blocked reaches memory on the device: 32-byte global reads and writes (256-bit accesses of
// sm_100), and the three four-entry windows of a thread in shared memory, laid out [window][entry][thread] so
// that a thread's 8-byte accesses always fall into its own pair of banks whatever window and entry it is at.
struct BlockedMem {
  uint2* win;   // &windows[0][0][threadIdx.x]; next entry / window kListThreads elements further
  __device__ __forceinline__ void load_window(int run, const WalkEntry* src) {
    unsigned v0, v1, v2, v3, v4, v5, v6, v7;
    asm volatile("ld.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3), "=r"(v4), "=r"(v5), "=r"(v6), "=r"(v7) : "l"(src));
    uint2* w = win + run * 4 * kListThreads;
    w[0] = make_uint2(v0, v1);
    w[kListThreads] = make_uint2(v2, v3);
    w[2 * kListThreads] = make_uint2(v4, v5);
    w[3 * kListThreads] = make_uint2(v6, v7);
  }
  __device__ __forceinline__ WalkEntry window(int run, int k) const { return win[(run * 4 + k) * kListThreads]; }
  __device__ __forceinline__ void store4(WalkEntry* dst, const WalkEntry (&e)[4]) const {
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(dst), "r"(e[0].x), "r"(e[0].y), "r"(e[1].x), "r"(e[1].y), "r"(e[2].x), "r"(e[2].y), "r"(e[3].x), "r"(e[3].y)
                 : "memory");
  }
  __device__ __forceinline__ void store1(WalkEntry* dst, const WalkEntry& e) const { *dst = e; }
};

// One piece of a merge that `parts` neighbouring lanes share (parts a power of two up to 32, so the lanes of one
// merge sit in one warp): every lane finds its own cut by binary search, takes the next lane's as its end and
// merges what lies between. All 32 lanes of the warp must call this, n[] being zero for lanes without work.
__device__ __forceinline__ void merge_piece(const WalkEntry* const* run, const int* n, const uint32_t* off, int part,
                                            int parts, WalkEntry* dst, BlockedMem& mem) {
  int cut[3], end[3];
  merge3_cut<WalkEntry>(run, n, part, parts, cut);
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    end[k] = __shfl_down_sync(0xffffffffu, cut[k], 1);
    if (part == parts - 1) end[k] = n[k];
  }
  const int count = (end[0] - cut[0]) + (end[1] - cut[1]) + (end[2] - cut[2]);
  merge3_runs_blocked_range<WalkEntry, BlockedMem>(run[0], run[1], run[2], off[0], off[1], off[2], cut[0], cut[1],
                                                   cut[2], count, dst, mem);
}

// One thread (SPLIT: `parts` neighbouring threads, each a piece) per (b, h, nw): merge of the pixel runs
// (b, h, nw - pad_left + kw), kw < Kw, columns outside the image being empty. Entry offsets gain kw*C*J.
template <bool SPLIT>
__global__ void __launch_bounds__(kListThreads)
snn_row_runs_kernel(const Geometry g, const WalkEntry* __restrict__ pix, const int* __restrict__ pix_n, int pix_stride,
                    WalkEntry* __restrict__ rows, int* __restrict__ rows_n, int row_stride, int parts_log2) {
  __shared__ uint2 windows[3 * 4 * kListThreads];
  BlockedMem mem = {windows + threadIdx.x};
  const int items = g.B * g.H * g.Nw;
  const int thread = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = SPLIT ? (thread >> parts_log2) : thread;
  const bool valid = t < items;
  if (!SPLIT && !valid) return;
  const int nw = t % g.Nw;
  const int bh = t / g.Nw;                            // b*H + h
  const WalkEntry* run[3] = {g_empty_run, g_empty_run, g_empty_run};
  uint32_t off[3] = {0u, 0u, 0u};
  int n[3] = {0, 0, 0};
#pragma unroll
  for (int kw = 0; kw < 3; ++kw) {
    const int wc = nw - g.pad_left + kw;
    if (valid && kw < g.Kw && wc >= 0 && wc < g.W) {
      const int p = bh * g.W + wc;
      run[kw] = pix + (size_t)p * pix_stride;
      n[kw] = __ldg(pix_n + p);
    }
    off[kw] = (uint32_t)kw * (uint32_t)g.C * (uint32_t)g.J;
  }
  const int total = n[0] + n[1] + n[2];
  WalkEntry* dst = rows + (size_t)(valid ? t : 0) * row_stride;
  if (SPLIT) {
    const int part = thread & ((1 << parts_log2) - 1);
    merge_piece(run, n, off, part, 1 << parts_log2, dst, mem);
    if (valid && part == 0) {
      dst[total] = make_uint2(kRunEndBits, 0u);
      rows_n[t] = total;
    }
  } else {
    merge3_runs_blocked<WalkEntry, BlockedMem>(run[0], run[1], run[2], off[0], off[1], off[2], total, dst, true, mem);
    rows_n[t] = total;
  }
}

// One thread (SPLIT: `parts` neighbouring threads, each a piece) per receptive field r = (b*Nh + nh)*Nw + nw:
// merge of the row runs (b, nh - pad_top + kh, nw), kh < Kh, rows outside the image being empty. Entry offsets
// gain kh*Kw*C*J.
template <bool SPLIT>
__global__ void __launch_bounds__(kListThreads)
snn_field_lists_kernel(const Geometry g, const WalkEntry* __restrict__ rows, const int* __restrict__ rows_n,
                       int row_stride, WalkEntry* __restrict__ lists, int* __restrict__ nvalid, int istride,
                       int parts_log2) {
  __shared__ uint2 windows[3 * 4 * kListThreads];
  BlockedMem mem = {windows + threadIdx.x};
  const int thread = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = SPLIT ? (thread >> parts_log2) : thread;
  const bool valid = r < g.R;
  if (!SPLIT && !valid) return;
  const int nw = r % g.Nw;
  const int t0 = r / g.Nw;
  const int nh = t0 % g.Nh;
  const int b = t0 / g.Nh;
  const WalkEntry* run[3] = {g_empty_run, g_empty_run, g_empty_run};
  uint32_t off[3] = {0u, 0u, 0u};
  int n[3] = {0, 0, 0};
#pragma unroll
  for (int kh = 0; kh < 3; ++kh) {
    const int h = nh - g.pad_top + kh;
    if (valid && kh < g.Kh && h >= 0 && h < g.H) {
      const int t = (b * g.H + h) * g.Nw + nw;
      run[kh] = rows + (size_t)t * row_stride;
      n[kh] = __ldg(rows_n + t);
    }
    off[kh] = (uint32_t)kh * (uint32_t)g.Kw * (uint32_t)g.C * (uint32_t)g.J;
  }
  const int total = n[0] + n[1] + n[2];
  WalkEntry* dst = lists + (size_t)(valid ? r : 0) * istride;
  if (SPLIT) {
    const int part = thread & ((1 << parts_log2) - 1);
    merge_piece(run, n, off, part, 1 << parts_log2, dst, mem);
    if (valid && part == 0) nvalid[r] = total;
  } else {
    merge3_runs_blocked<WalkEntry, BlockedMem>(run[0], run[1], run[2], off[0], off[1], off[2], total, dst, false, mem);
    nvalid[r] = total;
  }
}

// entries per pixel run and per row run: room for the terminator, rounded up to four entries (32 bytes)
int pixel_stride(const Geometry& g) { return (g.C + 1 + 3) & ~3; }
int row_stride(const Geometry& g) { return (g.Kw * g.C + 1 + 3) & ~3; }
size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

struct MergeScratch { size_t pix, pix_n, rows, rows_n, total; };
MergeScratch merge_scratch(const Geometry& g) {
  MergeScratch m;
  const size_t npix = (size_t)g.B * g.H * g.W, nrow = (size_t)g.B * g.H * g.Nw;
  m.pix = 0;
  m.pix_n = m.pix + align256(npix * pixel_stride(g) * sizeof(WalkEntry));
  m.rows = m.pix_n + align256(npix * sizeof(int));
  m.rows_n = m.rows + align256(nrow * row_stride(g) * sizeof(WalkEntry));
  m.total = m.rows_n + align256(nrow * sizeof(int));
  return m;
}

}  // namespace

bool merge_lists_supported(const Geometry& g) {
  return merge_lists_shape_ok(g) && g.Sh == 1 && g.Sw == 1;
}

bool merge_lists_shape_ok(const Geometry& g) {
  if (!g.is_conv) return false;
  if (g.Kh < 1 || g.Kh > 3 || g.Kw < 1 || g.Kw > 3 || g.Kh * g.Kw < 2) return false;
  if (g.C < 16 || g.C > 512) return false;            // fewer channels: the per-pixel warps would idle; more: registers
  // every intermediate index stays inside 32 bits
  if ((long long)g.B * g.H * g.W * pixel_stride(g) > 0x7fffffffLL) return false;
  if ((long long)g.B * g.H * g.Nw * row_stride(g) > 0x7fffffffLL) return false;
  return true;
}

size_t merge_lists_bytes(const Geometry& g) { return merge_scratch(g).total; }

// pieces per merge (as a power of two): enough that the merge kernels have about 768 threads per SM to run, and
// two pieces where one per merge would leave the last quarter of the thread slots empty (measured: 12.5 k to 65 k
// merges are fastest with about 100 k to 130 k threads, 200 k merges in two pieces, 262 k in one)
int merge_split_log2(int items, const LaunchInfo& li) {
  int lg = 0;
  while (lg < 4 && ((long)items << lg) < (long)li.num_sms * 768) ++lg;
  if (lg == 0 && items < li.num_sms * 1536) lg = 1;
  return lg;
}

int launch_merge_lists(const Geometry& g, const float* x, WalkEntry* lists, int* nvalid, int istride,
                       void* scratch, int split_log2, const LaunchInfo& li, cudaStream_t s) {
  const MergeScratch m = merge_scratch(g);
  unsigned char* base = static_cast<unsigned char*>(scratch);
  WalkEntry* pix = reinterpret_cast<WalkEntry*>(base + m.pix);
  int* pix_n = reinterpret_cast<int*>(base + m.pix_n);
  WalkEntry* rows = reinterpret_cast<WalkEntry*>(base + m.rows);
  int* rows_n = reinterpret_cast<int*>(base + m.rows_n);
  const int npix = g.B * g.H * g.W;
  const int ps = pixel_stride(g), rs = row_stride(g);
  const float maxcomp = g.maxv - 0.1f;

  long grid = ((long)npix + kPixelWarps - 1) / kPixelWarps;
  const long cap = (long)li.num_sms * 8;
  if (grid > cap) grid = cap;
  const int epl = (g.C + 31) / 32;
  if (epl <= 1) snn_pixel_runs_kernel<1><<<(int)grid, kPixelWarps * 32, 0, s>>>(x, npix, g.C, g.J, maxcomp, pix, pix_n, ps);
  else if (epl <= 2) snn_pixel_runs_kernel<2><<<(int)grid, kPixelWarps * 32, 0, s>>>(x, npix, g.C, g.J, maxcomp, pix, pix_n, ps);
  else if (epl <= 4) snn_pixel_runs_kernel<4><<<(int)grid, kPixelWarps * 32, 0, s>>>(x, npix, g.C, g.J, maxcomp, pix, pix_n, ps);
  else if (epl <= 8) snn_pixel_runs_kernel<8><<<(int)grid, kPixelWarps * 32, 0, s>>>(x, npix, g.C, g.J, maxcomp, pix, pix_n, ps);
  else snn_pixel_runs_kernel<16><<<(int)grid, kPixelWarps * 32, 0, s>>>(x, npix, g.C, g.J, maxcomp, pix, pix_n, ps);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return E_CUDA;

  const int nrow = g.B * g.H * g.Nw;
  int lg = split_log2 >= 0 ? (split_log2 > 5 ? 5 : split_log2) : merge_split_log2(nrow, li);
  if (((long)nrow << lg) > 0x7fffffffL - kListThreads) lg = 0;
  if (lg == 0)
    snn_row_runs_kernel<false><<<(nrow + kListThreads - 1) / kListThreads, kListThreads, 0, s>>>(g, pix, pix_n, ps, rows, rows_n, rs, 0);
  else
    snn_row_runs_kernel<true><<<(int)((((long)nrow << lg) + kListThreads - 1) / kListThreads), kListThreads, 0, s>>>(g, pix, pix_n, ps, rows, rows_n, rs, lg);
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return E_CUDA;

  lg = split_log2 >= 0 ? (split_log2 > 5 ? 5 : split_log2) : merge_split_log2(g.R, li);
  if (((long)g.R << lg) > 0x7fffffffL - kListThreads) lg = 0;
  if (lg == 0)
    snn_field_lists_kernel<false><<<(g.R + kListThreads - 1) / kListThreads, kListThreads, 0, s>>>(g, rows, rows_n, rs, lists, nvalid, istride, 0);
  else
    snn_field_lists_kernel<true><<<(int)((((long)g.R << lg) + kListThreads - 1) / kListThreads), kListThreads, 0, s>>>(g, rows, rows_n, rs, lists, nvalid, istride, lg);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

bool small_rows_supported(const Geometry& g) {
  if (g.I < 1 || g.I > 256) return false;
  if (g.is_conv && (g.Kh > 255 || g.Kw > 255)) return false;
  return true;
}

int launch_small_rows(const Geometry& g, const float* x, WalkEntry* lists, int* nvalid, int istride,
                      const LaunchInfo& li, cudaStream_t s) {
  long grid = ((long)g.R + kPixelWarps - 1) / kPixelWarps;
  const long cap = (long)li.num_sms * 8;
  if (grid > cap) grid = cap;
  const int epl = (g.I + 31) / 32;
  switch (epl) {   // 3, 5, 6, 7 keys per lane: the block network (a bitonic one would round them up to 4 and 8)
    case 1: snn_small_rows_kernel<1><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 2: snn_small_rows_kernel<2><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 3: snn_small_rows_kernel<3><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 4: snn_small_rows_kernel<4><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 5: snn_small_rows_kernel<5><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 6: snn_small_rows_kernel<6><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    case 7: snn_small_rows_kernel<7><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
    default: snn_small_rows_kernel<8><<<(int)grid, kPixelWarps * 32, 0, s>>>(g, x, lists, nvalid, istride); break;
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OK : E_CUDA;
}

}  // namespace snntc
