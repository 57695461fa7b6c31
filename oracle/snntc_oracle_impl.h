/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the SNN-TC operator semantics.
 *
 * This header is included twice by snntc_oracle.c: once with ACC = float (every
 * sum is carried in fp32 in the same order as the reference GPU kernels, products
 * fused into the sum with fmaf exactly where nvcc fuses them) and once with
 * ACC = double (a high-precision evaluation used to decide which outputs are
 * ill-conditioned and as the tolerance anchor for gradients).
 *
 * It restates, in plain C, what the reference GPU kernels compute:
 *   forward  : snntc/snnfc_kernels.cu.cc:19-71  (and its clone snntc/snncv_kernels.cu.cc:19-72)
 *   backward : snntc/snnfcgrad_kernels.cu.cc:15-133, snntc/snncvgrad_kernels.cu.cc:15-161
 *   patches  : snntc/snncvgrad_kernels.cu.cc:36-43 (row r = (b*Nh+nh)*Nw+nw, tap i = (kh*Kw+kw)*C+c)
 * Nothing here is shipped or timed as the product.
 */

#ifndef ACC
#error "define ACC and SUFFIX before including"
#endif

#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)
#define FN(name) CAT(name, SUFFIX)

#if ACC_IS_DOUBLE
#define FMA_ACC(a, b, c) ((a) * (b) + (c))
#else
#define FMA_ACC(a, b, c) fmaf((a), (b), (c))
#endif

/* sign-safe "ysum/wsum > c" without a division (snnfc_kernels.cu.cc:36-38, 53-55) */
static inline int FN(ratio_gt)(ACC ysum, ACC wsum, ACC c) {
  ACC wa = wsum, ya = ysum;
  if (wa < 0) { wa = -wa; ya = -ya; }
  return ya > wa * c;
}
/* sign-safe "ysum/wsum <= c" (snnfc_kernels.cu.cc:46-48) */
static inline int FN(ratio_le)(ACC ysum, ACC wsum, ACC c) {
  ACC wa = wsum, ya = ysum;
  if (wa < 0) { wa = -wa; ya = -ya; }
  return ya <= c * wa;
}

/* A decision "ysum/wsum vs c" counts as ill-conditioned when |ysum - c*wsum| is within tol of the
 * compared magnitudes (plus a small share of c*(theta+sum|w|), the scale of the fp32 rounding noise). */
static inline int FN(near_tie)(double ysum, double wsum, double c, double asum, double tol) {
  return fabs(ysum - c * wsum) < tol * (fabs(ysum) + fabs(c * wsum)) + 0.02 * tol * fabs(c) * asum;
}

/*
 * One row (dense sample or conv patch) through the forward walk for all J outputs.
 * xs[k]   : the row's inputs sorted ascending, ord[k] their source index (ties by index)
 * y,inv   : outputs (spike value or MAX; 1/(sum w - theta) or 0)
 * kcount  : optional, number of inputs consumed before the exit
 * illc    : optional (double build only), 1 where a decision on the path to the exit
 *           was closer than `tol` to flipping (see near_tie)
 * cond    : optional, (theta+sum|w|)/|sum w - theta| of a fired output: how much fp32 rounding of the
 *           sums is amplified in y; 0 where the output did not fire
 */
static void FN(row_forward)(const float* xs, const int* ord, int I, const float* w, int J,
                            float maxv, float theta, float biasvolt,
                            ACC* y, ACC* inv, int* kcount, unsigned char* illc, double tol, double* cond) {
  const ACC maxcomp = (ACC)maxv - (ACC)0.1f;
  for (int j = 0; j < J; ++j) {
    ACC wsum = -(ACC)theta, ysum = 0;
    double asum = fabs((double)theta);
    int armed = 0, k, bad = 0;
    if (biasvolt > 1e-8f) {
      ACC wb = (ACC)w[(size_t)I * J + j];
      wsum += wb;
      ysum = (ACC)biasvolt * wb;
      asum += fabs((double)wb);
      armed = FN(ratio_gt)(ysum, wsum, (ACC)biasvolt);
      if (illc && FN(near_tie)((double)ysum, (double)wsum, (double)biasvolt, asum, tol)) bad = 1;
    }
    for (k = 0; k < I; ++k) {
      ACC x = (ACC)xs[k];
      if (x > maxcomp) break;
      if (illc && FN(near_tie)((double)ysum, (double)wsum, (double)x, asum, tol)) bad = 1;
      if (armed && FN(ratio_le)(ysum, wsum, x)) break;
      ACC wk = (ACC)w[(size_t)ord[k] * J + j];
      wsum += wk;
      ysum = FMA_ACC(x, wk, ysum);
      asum += fabs((double)wk);
      armed = FN(ratio_gt)(ysum, wsum, x);
      if (illc && FN(near_tie)((double)ysum, (double)wsum, (double)x, asum, tol)) bad = 1;
    }
    ACC yo = (ACC)maxv, io = 0;
    if (armed) {
      io = (ACC)1 / wsum;
      yo = ysum * io;
      if (yo >= (ACC)maxv) { yo = (ACC)maxv; io = 0; }
      if (illc && fabs((double)wsum) < tol * asum) bad = 1;
    }
    y[j] = yo;
    inv[j] = io;
    if (kcount) kcount[j] = k;
    if (illc) illc[j] = (unsigned char)bad;
    if (cond) cond[j] = (armed && io != 0) ? asum / fabs((double)wsum) : 0.0;
  }
}

/* stable ascending sort of one row: values + source index (merge sort, ties keep index order) */
static void FN(sort_row)(const float* x, int I, float* xs, int* ord, float* tx, int* to) {
  for (int i = 0; i < I; ++i) { xs[i] = x[i]; ord[i] = i; }
  for (int width = 1; width < I; width *= 2) {
    for (int lo = 0; lo < I; lo += 2 * width) {
      int mid = lo + width < I ? lo + width : I, hi = lo + 2 * width < I ? lo + 2 * width : I;
      int a = lo, b = mid;
      for (int k = lo; k < hi; ++k) {
        if (a < mid && (b >= hi || xs[a] <= xs[b])) { tx[k] = xs[a]; to[k] = ord[a]; ++a; }
        else { tx[k] = xs[b]; to[k] = ord[b]; ++b; }
      }
    }
    memcpy(xs, tx, sizeof(float) * (size_t)I);
    memcpy(ord, to, sizeof(int) * (size_t)I);
  }
}

/* Forward over R rows given as a dense matrix rows[R,I]; out is [2R,J]-packed like the op. */
int FN(oracle_rows_forward)(const float* rows, const float* w, int R, int I, int J,
                            float maxv, float theta, float biasvolt,
                            ACC* y, ACC* inv, int* kcount, unsigned char* illc, double tol, double* cond) {
  float* xs = (float*)malloc(sizeof(float) * (size_t)(I > 0 ? I : 1) * 2);
  int* ord = (int*)malloc(sizeof(int) * (size_t)(I > 0 ? I : 1) * 2);
  if (!xs || !ord) { free(xs); free(ord); return -1; }
  for (int r = 0; r < R; ++r) {
    FN(sort_row)(rows + (size_t)r * I, I, xs, ord, xs + I, ord + I);
    FN(row_forward)(xs, ord, I, w, J, maxv, theta, biasvolt, y + (size_t)r * J, inv + (size_t)r * J,
                    kcount ? kcount + (size_t)r * J : 0, illc ? illc + (size_t)r * J : 0, tol,
                    cond ? cond + (size_t)r * J : 0);
  }
  free(xs); free(ord);
  return 0;
}

/*
 * Dense-row backward (snnfcgrad_kernels.cu.cc:56-65 for dX, :100-120 for dW).
 * g[R,J] upstream gradient of y, yv[R,J] forward spike values, iv[R,J] forward 1/(sum w - theta).
 * dx[R,I] (nullable), dw[(I+bias),J] accumulated in ACC; dw must be zeroed by the caller.
 * dx_abs / dw_abs (nullable, zeroed by the caller) receive the sum of |terms| of every element: the
 * scale against which fp32 summation error has to be judged.
 */
int FN(oracle_rows_backward)(const float* g, const float* rows, const float* w, const float* yv,
                             const float* iv, int R, int I, int J, float maxv, float biasvolt,
                             ACC* dx, ACC* dw, double* dx_abs, double* dw_abs) {
  const float maxcomp = maxv - 0.1f;
  const int bias = biasvolt > 1e-8f;
  for (int r = 0; r < R; ++r) {
    const float* xr = rows + (size_t)r * I;
    for (int j = 0; j < J; ++j) {
      float yj = yv[(size_t)r * J + j];
      if (yj > maxcomp) continue;
      ACC u = (ACC)(g[(size_t)r * J + j] * iv[(size_t)r * J + j]); /* product formed in fp32, as the reference does */
      for (int i = 0; i < I; ++i) {
        float x = xr[i];
        if (x > yj) continue;
        if (dx) dx[(size_t)r * I + i] = FMA_ACC(u, (ACC)w[(size_t)i * J + j], dx[(size_t)r * I + i]);
        if (dx_abs) dx_abs[(size_t)r * I + i] += fabs((double)u * (double)w[(size_t)i * J + j]);
        if (x > maxcomp) continue;
        dw[(size_t)i * J + j] = FMA_ACC((ACC)x - (ACC)yj, u, dw[(size_t)i * J + j]);
        if (dw_abs) dw_abs[(size_t)i * J + j] += fabs(((double)x - (double)yj) * (double)u);
      }
      if (bias && !(biasvolt > yj)) {
        dw[(size_t)I * J + j] = FMA_ACC((ACC)biasvolt - (ACC)yj, u, dw[(size_t)I * J + j]);
        if (dw_abs) dw_abs[(size_t)I * J + j] += fabs(((double)biasvolt - (double)yj) * (double)u);
      }
    }
  }
  return 0;
}

/* gather one conv patch row; taps outside the image read MAX (SNN_TC_Modules.py:147-161 pads with MAX) */
static void FN(gather_patch)(const float* x, int H, int W, int C, int Kh, int Kw, int Sh, int Sw,
                             int pt, int pl, int b, int nh, int nw, float maxv, float* row) {
  for (int kh = 0; kh < Kh; ++kh)
    for (int kw = 0; kw < Kw; ++kw) {
      int h = nh * Sh + kh - pt, ww = nw * Sw + kw - pl;
      float* dst = row + ((size_t)kh * Kw + kw) * C;
      if (h < 0 || h >= H || ww < 0 || ww >= W) { for (int c = 0; c < C; ++c) dst[c] = maxv; }
      else memcpy(dst, x + (((size_t)b * H + h) * W + ww) * C, sizeof(float) * (size_t)C);
    }
}

/* Conv forward on the UNPADDED NHWC input x[B,H,W,C] with pad_top/pad_left and output grid Nh x Nw. */
int FN(oracle_cv_forward)(const float* x, const float* w, int B, int H, int W, int C, int Kc,
                          int Kh, int Kw, int Sh, int Sw, int pt, int pl, int Nh, int Nw,
                          float maxv, float theta, float biasvolt,
                          ACC* y, ACC* inv, int* kcount, unsigned char* illc, double tol, double* cond) {
  int I = Kh * Kw * C;
  float* row = (float*)malloc(sizeof(float) * (size_t)I * 3);
  int* ord = (int*)malloc(sizeof(int) * (size_t)I * 2);
  if (!row || !ord) { free(row); free(ord); return -1; }
  size_t r = 0;
  for (int b = 0; b < B; ++b)
    for (int nh = 0; nh < Nh; ++nh)
      for (int nw = 0; nw < Nw; ++nw, ++r) {
        FN(gather_patch)(x, H, W, C, Kh, Kw, Sh, Sw, pt, pl, b, nh, nw, maxv, row);
        FN(sort_row)(row, I, row + I, ord, row + 2 * (size_t)I, ord + I);
        FN(row_forward)(row + I, ord, I, w, Kc, maxv, theta, biasvolt, y + r * Kc, inv + r * Kc,
                        kcount ? kcount + r * Kc : 0, illc ? illc + r * Kc : 0, tol, cond ? cond + r * Kc : 0);
      }
  free(row); free(ord);
  return 0;
}

/* Conv backward; dx is the UNPADDED [B,H,W,C] gradient (padding taps drop out), both dx and dw zeroed by caller. */
int FN(oracle_cv_backward)(const float* g, const float* x, const float* w, const float* yv, const float* iv,
                           int B, int H, int W, int C, int Kc, int Kh, int Kw, int Sh, int Sw,
                           int pt, int pl, int Nh, int Nw, float maxv, float biasvolt,
                           ACC* dx, ACC* dw, double* dx_abs, double* dw_abs) {
  const float maxcomp = maxv - 0.1f;
  const int bias = biasvolt > 1e-8f;
  const int I = Kh * Kw * C;
  size_t r = 0;
  for (int b = 0; b < B; ++b)
    for (int nh = 0; nh < Nh; ++nh)
      for (int nw = 0; nw < Nw; ++nw, ++r)
        for (int j = 0; j < Kc; ++j) {
          float yj = yv[r * Kc + j];
          if (yj > maxcomp) continue;
          ACC u = (ACC)(g[r * Kc + j] * iv[r * Kc + j]);
          for (int kh = 0; kh < Kh; ++kh)
            for (int kw = 0; kw < Kw; ++kw) {
              int h = nh * Sh + kh - pt, ww = nw * Sw + kw - pl;
              if (h < 0 || h >= H || ww < 0 || ww >= W) continue; /* MAX tap: x > y always */
              size_t xo = (((size_t)b * H + h) * W + ww) * C;
              size_t wo = ((size_t)kh * Kw + kw) * C;
              for (int c = 0; c < C; ++c) {
                float xv = x[xo + c];
                if (xv > yj) continue;
                if (dx) dx[xo + c] = FMA_ACC(u, (ACC)w[(wo + c) * Kc + j], dx[xo + c]);
                if (dx_abs) dx_abs[xo + c] += fabs((double)u * (double)w[(wo + c) * Kc + j]);
                if (xv > maxcomp) continue;
                dw[(wo + c) * Kc + j] = FMA_ACC((ACC)xv - (ACC)yj, u, dw[(wo + c) * Kc + j]);
                if (dw_abs) dw_abs[(wo + c) * Kc + j] += fabs(((double)xv - (double)yj) * (double)u);
              }
            }
          if (bias && !(biasvolt > yj)) {
            dw[(size_t)I * Kc + j] = FMA_ACC((ACC)biasvolt - (ACC)yj, u, dw[(size_t)I * Kc + j]);
            if (dw_abs) dw_abs[(size_t)I * Kc + j] += fabs(((double)biasvolt - (double)yj) * (double)u);
          }
        }
  return 0;
}

#undef FMA_ACC
#undef FN
#undef CAT
#undef CAT2
