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

}  // namespace snntc
