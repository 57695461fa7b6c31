// Sequential merge of up to three sorted runs of list entries, one thread per merge.
//
// A run is a sequence of entries (x = float bits of an input value, y = element offset of a weight row) in
// ascending order of x that ends with one extra entry whose x is +inf, so that a run that is used up shows a
// head that never wins while another run still has entries; no bounds are tested inside the loop. An empty
// run is any pointer to such a terminator. Inputs hold no NaN (the per-pixel sort drops them with the inputs
// that never spike) and every real entry is finite, so plain float comparisons order the heads.
//
// The function is plain C++ so that the same source can be compiled for the host by a unit test.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SNNTC_HD __host__ __device__ __forceinline__
#else
#define SNNTC_HD inline
#endif

namespace snntc {

SNNTC_HD float entry_value(uint32_t bits) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(bits);
#else
  union { uint32_t u; float f; } cv; cv.u = bits; return cv.f;
#endif
}

constexpr uint32_t kRunEndBits = 0x7f800000u;   // +inf

// Merges runs a, b, c (each terminated as described above) into dst[0 .. total), adding off_a / off_b / off_c
// to the y field of the entries taken from the respective run; ties go to the earlier run. `total` is the
// number of real entries of the three runs together. When `terminate` is set, dst[total] receives a
// terminator, so that dst is a run itself. Entries are written two at a time (16 bytes) where dst allows it:
// dst must be 16-byte aligned.
template <typename Entry, typename Entry2>
SNNTC_HD void merge3_runs(const Entry* __restrict__ a, const Entry* __restrict__ b, const Entry* __restrict__ c,
                          uint32_t off_a, uint32_t off_b, uint32_t off_c, int total, Entry* __restrict__ dst,
                          bool terminate) {
  Entry ha = a[0], hb = b[0], hc = c[0];
  uint32_t pa = 0, pb = 0, pc = 0;
  Entry pending;
  pending.x = 0; pending.y = 0;
  for (int k = 0; k < total; ++k) {
    const float fa = entry_value(ha.x), fb = entry_value(hb.x), fc = entry_value(hc.x);
    const bool sa = (fa <= fb) & (fa <= fc);
    const bool sb = !sa & (fb <= fc);
    Entry out;
    out.x = sa ? ha.x : (sb ? hb.x : hc.x);
    out.y = (sa ? ha.y : (sb ? hb.y : hc.y)) + (sa ? off_a : (sb ? off_b : off_c));
    const Entry* run = sa ? a : (sb ? b : c);
    const uint32_t pos = (sa ? pa : (sb ? pb : pc)) + 1u;
    const Entry next = run[pos];   // at worst the run's terminator
    if (sa) { ha = next; pa = pos; } else if (sb) { hb = next; pb = pos; } else { hc = next; pc = pos; }
    if (k & 1) {
      Entry2 two;
      two.x = pending.x; two.y = pending.y; two.z = out.x; two.w = out.y;
      *reinterpret_cast<Entry2*>(dst + (k - 1)) = two;
    } else {
      pending = out;
    }
  }
  if (total & 1) dst[total - 1] = pending;
  if (terminate) {
    Entry end;
    end.x = kRunEndBits; end.y = 0;
    dst[total] = end;
  }
}

// The same merge moving four entries (32 bytes) per memory transaction: a thread that reads and writes 8 bytes at
// a time touches a different 32-byte sector with every access, so a warp's load or store is 32 sector
// transactions for 256 useful bytes. Here every run is read through a four-entry window (refilled by one 32-byte
// read whenever the position crosses a multiple of four) and the output leaves four entries at a time.
//   Mem::load_window(run, src)   copies entries src[0..4) into window `run` (0..2); src is 32-byte aligned
//   Mem::window(run, k)          entry k of window `run`
//   Mem::store4(dst, e)          writes e[0..4) to dst[0..4); dst is 32-byte aligned
// Runs, dst and the empty run must be 32-byte aligned and readable / writable up to the next multiple of four
// entries past their terminator (past `total` for dst): the last group is written whole, whatever lies behind
// `total` in it is unspecified.
template <typename Entry, typename Mem>
SNNTC_HD void merge3_runs_blocked(const Entry* __restrict__ a, const Entry* __restrict__ b, const Entry* __restrict__ c,
                                  uint32_t off_a, uint32_t off_b, uint32_t off_c, int total, Entry* __restrict__ dst,
                                  bool terminate, Mem& mem) {
  mem.load_window(0, a);
  mem.load_window(1, b);
  mem.load_window(2, c);
  Entry ha = mem.window(0, 0), hb = mem.window(1, 0), hc = mem.window(2, 0);
  uint32_t pa = 0, pb = 0, pc = 0;
  for (int k0 = 0; k0 < total; k0 += 4) {
    Entry out[4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int u = 0; u < 4; ++u) {
      out[u].x = 0; out[u].y = 0;
      if (k0 + u < total) {
        const float fa = entry_value(ha.x), fb = entry_value(hb.x), fc = entry_value(hc.x);
        const bool sa = (fa <= fb) & (fa <= fc);
        const bool sb = !sa & (fb <= fc);
        out[u].x = sa ? ha.x : (sb ? hb.x : hc.x);
        out[u].y = (sa ? ha.y : (sb ? hb.y : hc.y)) + (sa ? off_a : (sb ? off_b : off_c));
        const Entry* run = sa ? a : (sb ? b : c);
        const int which = sa ? 0 : (sb ? 1 : 2);
        const uint32_t pos = (sa ? pa : (sb ? pb : pc)) + 1u;
        if ((pos & 3u) == 0u) mem.load_window(which, run + pos);
        const Entry next = mem.window(which, (int)(pos & 3u));   // at worst the run's terminator
        if (sa) { ha = next; pa = pos; } else if (sb) { hb = next; pb = pos; } else { hc = next; pc = pos; }
      }
    }
    mem.store4(dst + k0, out);
  }
  if (terminate) {
    Entry end;
    end.x = kRunEndBits; end.y = 0;
    dst[total] = end;
  }
}

// Number of entries of `run` (n real entries, ascending) whose value is < v (or_equal = false) or <= v (true).
template <typename Entry>
SNNTC_HD int run_bound(const Entry* __restrict__ run, int n, float v, bool or_equal) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const float f = entry_value(run[mid].x);
    const bool before = or_equal ? (f <= v) : (f < v);
    if (before) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// Splits the merge of three runs into `parts` pieces by VALUE: cut `part` (0 .. parts) is the triple of positions
// (pos[0], pos[1], pos[2]) such that the merged sequence up to the cut consists of exactly a[0..pos[0]),
// b[0..pos[1]) and c[0..pos[2]). The cut values are taken from the longest run at equal steps of its length; in the
// other runs the cut falls behind the entries equal to the cut value for a run that wins ties against the longest
// one (an earlier run) and in front of them for a later run, which is where the sequential merge puts them.
// Cut 0 is (0,0,0), cut `parts` is (n[0], n[1], n[2]).
template <typename Entry>
SNNTC_HD void merge3_cut(const Entry* const* run, const int* n, int part, int parts, int* pos) {
  if (part <= 0) { pos[0] = pos[1] = pos[2] = 0; return; }
  if (part >= parts) { pos[0] = n[0]; pos[1] = n[1]; pos[2] = n[2]; return; }
  int longest = 0;
  if (n[1] > n[longest]) longest = 1;
  if (n[2] > n[longest]) longest = 2;
  const int ip = (int)(((long long)n[longest] * part) / parts);
  if (n[longest] == 0) { pos[0] = pos[1] = pos[2] = 0; return; }
  const float v = entry_value(run[longest][ip].x);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int k = 0; k < 3; ++k) {
    if (k == longest) pos[k] = ip;
    else pos[k] = run_bound<Entry>(run[k], n[k], v, k < longest);
  }
}

// merge3_runs_blocked for one piece of a split merge: starts with the heads at a[pa], b[pb], c[pc], produces
// `count` entries and writes them to dst[d0 .. d0+count), d0 = pa+pb+pc. dst itself (not dst+d0) is 32-byte aligned;
// groups of four entries that belong to this piece in full leave as one 32-byte store, the entries in front of
// the first and behind the last such group one by one (the rest of those groups belongs to the neighbouring
// pieces). Additionally needs Mem::store1(dst, e). Writes no terminator.
template <typename Entry, typename Mem>
SNNTC_HD void merge3_runs_blocked_range(const Entry* __restrict__ a, const Entry* __restrict__ b,
                                        const Entry* __restrict__ c, uint32_t off_a, uint32_t off_b, uint32_t off_c,
                                        int pa_, int pb_, int pc_, int count, Entry* __restrict__ dst, Mem& mem) {
  uint32_t pa = (uint32_t)pa_, pb = (uint32_t)pb_, pc = (uint32_t)pc_;
  mem.load_window(0, a + (pa & ~3u));
  mem.load_window(1, b + (pb & ~3u));
  mem.load_window(2, c + (pc & ~3u));
  Entry ha = mem.window(0, (int)(pa & 3u)), hb = mem.window(1, (int)(pb & 3u)), hc = mem.window(2, (int)(pc & 3u));
  int k = pa_ + pb_ + pc_;
  const int kend = k + count;
#define SNNTC_MERGE_STEP(OUT)                                                                      \
  {                                                                                                \
    const float fa = entry_value(ha.x), fb = entry_value(hb.x), fc = entry_value(hc.x);            \
    const bool sa = (fa <= fb) & (fa <= fc);                                                       \
    const bool sb = !sa & (fb <= fc);                                                              \
    (OUT).x = sa ? ha.x : (sb ? hb.x : hc.x);                                                      \
    (OUT).y = (sa ? ha.y : (sb ? hb.y : hc.y)) + (sa ? off_a : (sb ? off_b : off_c));              \
    const Entry* run = sa ? a : (sb ? b : c);                                                      \
    const int which = sa ? 0 : (sb ? 1 : 2);                                                       \
    const uint32_t pos = (sa ? pa : (sb ? pb : pc)) + 1u;                                          \
    if ((pos & 3u) == 0u) mem.load_window(which, run + pos);                                       \
    const Entry next = mem.window(which, (int)(pos & 3u));                                         \
    if (sa) { ha = next; pa = pos; } else if (sb) { hb = next; pb = pos; } else { hc = next; pc = pos; } \
  }
  while (k < kend && (k & 3)) {
    Entry e;
    SNNTC_MERGE_STEP(e)
    mem.store1(dst + k, e);
    ++k;
  }
  for (; k + 4 <= kend; k += 4) {
    Entry out[4];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int u = 0; u < 4; ++u) SNNTC_MERGE_STEP(out[u])
    mem.store4(dst + k, out);
  }
  while (k < kend) {
    Entry e;
    SNNTC_MERGE_STEP(e)
    mem.store1(dst + k, e);
    ++k;
  }
#undef SNNTC_MERGE_STEP
}

}  // namespace snntc
