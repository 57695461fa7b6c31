/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the four SNN-TC operators.
 *
 * Plain-C restatement of the reference GPU kernels' arithmetic (see snntc_oracle_impl.h for the
 * file:line map). Two instantiations are exported:
 *   *_f32 : fp32 sums in the reference's order (what a faithful GPU kernel should reproduce)
 *   *_f64 : double sums (tolerance anchor; also flags ill-conditioned fire decisions)
 * Only tests, the smoke check and the bench's CPU-baseline leg may load this library; the product
 * never does.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define ACC float
#define ACC_IS_DOUBLE 0
#define SUFFIX _f32
#include "snntc_oracle_impl.h"
#undef ACC
#undef ACC_IS_DOUBLE
#undef SUFFIX

#define ACC double
#define ACC_IS_DOUBLE 1
#define SUFFIX _f64
#include "snntc_oracle_impl.h"
#undef ACC
#undef ACC_IS_DOUBLE
#undef SUFFIX

/* 2x2-style earliest-spike pooling used between conv layers (SNN_TC_Modules.py:216-246):
 * pad with padvalue, then min over each Kh x Kw window with stride (Sh,Sw), VALID. Also returns the
 * flat input index of the winner (first minimum in (kh,kw) scan order; -1 if the winner is padding). */
int oracle_minpool(const float* x, int B, int H, int W, int C, int Kh, int Kw, int Sh, int Sw,
                   int pt, int pl, int Nh, int Nw, float padvalue, float* y, int* arg) {
  for (int b = 0; b < B; ++b)
    for (int nh = 0; nh < Nh; ++nh)
      for (int nw = 0; nw < Nw; ++nw)
        for (int c = 0; c < C; ++c) {
          float best = 0; int bi = -1, first = 1;
          for (int kh = 0; kh < Kh; ++kh)
            for (int kw = 0; kw < Kw; ++kw) {
              int h = nh * Sh + kh - pt, w = nw * Sw + kw - pl;
              float v = padvalue; int idx = -1;
              if (h >= 0 && h < H && w >= 0 && w < W) { idx = ((b * H + h) * W + w) * C + c; v = x[idx]; }
              if (first || v < best) { best = v; bi = idx; first = 0; }
            }
          size_t o = (((size_t)b * Nh + nh) * Nw + nw) * C + c;
          y[o] = best;
          if (arg) arg[o] = bi;
        }
  return 0;
}
