// The pieces of a training step that sit around the four SNN-TC operators in the reference's example
// trainers, as single kernels over flat fp32 buffers:
//   - input encoding      x = exp(scale * (1 - p))  or  exp(scale * p)            (snntc-mnist.py:75, snntc-cifar10.py)
//   - loss                mean softmax cross-entropy on the NEGATED spike times, its gradient and the
//                         arg-min accuracy count                                    (SNN_TC_Modules.py:286-288, snntc-mnist.py:82)
//   - weight cost         K * mean_j max(0, 1 - sum_i w_ij) + K2 * mean(w^2) and its gradient   (snntc-mnist.py:55-59)
//   - optimiser           Adam and SGD with momentum in the Keras formulation, reading the (all-reduced)
//                         gradient bucket in place                                  (snntc-mnist.py:70, snntc-imagenet.py:238)
// The reference runs these as TensorFlow graph ops; nothing here has native code in the reference.
#include "../../include/snntc_b200.h"

#include <cuda_runtime.h>
#include <math_constants.h>

namespace snntc { void count_launch(int n = 1); }

namespace {

int grid_for(size_t n, int per_block = 256) {
  size_t b = (n + per_block - 1) / per_block;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  return (int)b;
}

__global__ void encode_kernel(const float* __restrict__ p, float* __restrict__ x, size_t n, float scale, int one_minus) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const float v = __ldg(p + e);
    x[e] = expf(scale * (one_minus ? 1.0f - v : v));
  }
}

// One warp per sample: logits z = -y. loss_b = logsumexp(z) - z[label]; grad_y = -(softmax(z) - onehot) * gscale.
// sums[0] += loss_b * lscale, sums[1] += (argmin_j y == label). Ties in the arg-min go to the lowest index,
// as tf.argmin does.
__global__ void loss_ce_kernel(const float* __restrict__ y, const long long* __restrict__ labels, float* __restrict__ grad,
                               float* __restrict__ sums, int B, int J, float lscale, float gscale) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  float loss_acc = 0.f, hit_acc = 0.f;
  for (int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < B; b += warps) {
    const float* row = y + (size_t)b * J;
    float zmax = -CUDART_INF_F;
    int amin = 0x7fffffff;
    float ymin = CUDART_INF_F;
    for (int j = lane; j < J; j += 32) {
      const float v = __ldg(row + j);
      zmax = fmaxf(zmax, -v);
      if (v < ymin) { ymin = v; amin = j; }
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
      zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, d));
      const float oy = __shfl_xor_sync(0xffffffffu, ymin, d);
      const int oa = __shfl_xor_sync(0xffffffffu, amin, d);
      if (oy < ymin || (oy == ymin && oa < amin)) { ymin = oy; amin = oa; }
    }
    float se = 0.f;
    for (int j = lane; j < J; j += 32) se += expf(-__ldg(row + j) - zmax);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) se += __shfl_xor_sync(0xffffffffu, se, d);
    const float lse_rel = logf(se);   // logsumexp(z) - zmax: the loss is lse_rel + (zmax - z[label]), never lse itself,
                                      // which would lose the small term beside a large |zmax| (all outputs at MAX)
    const int lab = (int)labels[b];
    const float inv = 1.0f / se;
    if (grad != nullptr) {
      for (int j = lane; j < J; j += 32) {
        const float sm = expf(-__ldg(row + j) - zmax) * inv;
        grad[(size_t)b * J + j] = -(sm - (j == lab ? 1.0f : 0.0f)) * gscale;
      }
    }
    if (lane == 0) {
      const float zl = (lab >= 0 && lab < J) ? -__ldg(row + lab) : zmax;
      loss_acc += (lse_rel + (zmax - zl)) * lscale;
      hit_acc += (amin == lab) ? 1.0f : 0.0f;
    }
  }
  if (lane == 0) {
    if (loss_acc != 0.f) atomicAdd(sums, loss_acc);
    if (hit_acc != 0.f) atomicAdd(sums + 1, hit_acc);
  }
}

// column sums of w[rows, J] into colsum[J] (zeroed by the caller) and sum of squares into sq[0]
__global__ void wcost_sums_kernel(const float* __restrict__ w, float* __restrict__ colsum, float* __restrict__ sq,
                                  int rows, int J, int rows_per_block) {
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float s2 = 0.f;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < J; j += gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = r0; r < r1; ++r) {
      const float v = __ldg(w + (size_t)r * J + j);
      s += v;
      s2 = fmaf(v, v, s2);
    }
    atomicAdd(colsum + j, s);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, d);
  if ((threadIdx.x & 31) == 0 && s2 != 0.f) atomicAdd(sq, s2);
}

// cost[0] += K * mean_j max(0, 1 - colsum_j) + K2 * sq / (rows*J)   (block 0, thread-serial over a small J is
// avoided: every block adds its share), gw[i,j] += -K/J * [1 - colsum_j > 0] + 2*K2/(rows*J) * w[i,j]
__global__ void wcost_apply_kernel(const float* __restrict__ w, const float* __restrict__ colsum,
                                   const float* __restrict__ sq, float* __restrict__ gw, float* __restrict__ cost,
                                   int rows, int J, float K, float K2) {
  const size_t n = (size_t)rows * J;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const float a = -K / (float)J, b2 = 2.0f * K2 / (float)n;
  if (gw != nullptr) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
      const int j = (int)(e % J);
      const float hinge = (1.0f - __ldg(colsum + j)) > 0.f ? a : 0.f;
      gw[e] += hinge + b2 * __ldg(w + e);
    }
  }
  if (cost != nullptr) {
    float c = 0.f;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < (size_t)J; j += stride)
      c += fmaxf(0.f, 1.0f - __ldg(colsum + j));
    c *= K / (float)J;
    if (blockIdx.x == 0 && threadIdx.x == 0) c += K2 * __ldg(sq) / (float)n;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
    if ((threadIdx.x & 31) == 0 && c != 0.f) atomicAdd(cost, c);
  }
}

// Keras Adam: lr_t = lr * sqrt(1 - b2^t) / (1 - b1^t); m += (g - m)(1 - b1); v += (g^2 - v)(1 - b2);
// w -= lr_t * m / (sqrt(v) + eps). The step count t lives on the device (step[0] = steps taken so far), so that
// a captured CUDA graph replays with the count advancing; a one-thread kernel increments it after the update.
__global__ void adam_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                            size_t n, float lr, float b1, float b2, float eps, float gscale,
                            const int* __restrict__ step) {
  const int t = __ldg(step) + 1;
  const float c1 = 1.0f - powf(b1, (float)t), c2 = 1.0f - powf(b2, (float)t);
  const float lrt = lr * sqrtf(c2) / c1;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const float ge = __ldg(g + e) * gscale;
    const float me = m[e] + (ge - m[e]) * (1.0f - b1);
    const float ve = v[e] + (ge * ge - v[e]) * (1.0f - b2);
    m[e] = me;
    v[e] = ve;
    w[e] -= lrt * me / (sqrtf(ve) + eps);
  }
}
__global__ void step_inc_kernel(int* step) { *step += 1; }

// Keras SGD with momentum: vel = momentum * vel - lr * g; w += vel
__global__ void sgdm_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ vel, size_t n,
                            float lr, float momentum, float gscale) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const float ve = momentum * vel[e] - lr * (__ldg(g + e) * gscale);
    vel[e] = ve;
    w[e] += ve;
  }
}

int done() {
  snntc::count_launch();
  return cudaGetLastError() == cudaSuccess ? SNNTC_OK : SNNTC_E_CUDA;
}

}  // namespace

extern "C" {

int snntc_encode(const float* p, float* x, size_t n, float scale, int one_minus, void* stream) {
  if (!p || !x) return SNNTC_E_NULL;
  if (n == 0) return SNNTC_OK;
  encode_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(p, x, n, scale, one_minus);
  return done();
}

int snntc_loss_ce(const float* y, const long long* labels, float* grad, float* sums2, int B, int J,
                  float loss_scale, float grad_scale, void* stream) {
  if (!y || !labels || !sums2) return SNNTC_E_NULL;
  if (B <= 0 || J <= 0) return SNNTC_E_SHAPE;
  loss_ce_kernel<<<grid_for((size_t)B * 32), 256, 0, (cudaStream_t)stream>>>(y, labels, grad, sums2, B, J, loss_scale,
                                                                            grad_scale);
  return done();
}

size_t snntc_weight_cost_workspace_bytes(int J) { return ((size_t)J + 1) * sizeof(float); }

int snntc_weight_cost(const float* w, float* gw, float* cost, int rows, int J, float K, float K2,
                      void* workspace, size_t workspace_bytes, void* stream) {
  if (!w || !workspace) return SNNTC_E_NULL;
  if (rows <= 0 || J <= 0) return SNNTC_E_SHAPE;
  if (workspace_bytes < snntc_weight_cost_workspace_bytes(J)) return SNNTC_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  float* colsum = static_cast<float*>(workspace);
  float* sq = colsum + J;
  if (cudaMemsetAsync(workspace, 0, snntc_weight_cost_workspace_bytes(J), s) != cudaSuccess) return SNNTC_E_CUDA;
  const int rpb = 64;
  dim3 grid((J + 255) / 256, (rows + rpb - 1) / rpb);
  wcost_sums_kernel<<<grid, 256, 0, s>>>(w, colsum, sq, rows, J, rpb);
  if (done() != SNNTC_OK) return SNNTC_E_CUDA;
  wcost_apply_kernel<<<grid_for((size_t)rows * J), 256, 0, s>>>(w, colsum, sq, gw, cost, rows, J, K, K2);
  return done();
}

int snntc_adam_step(float* w, const float* g, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                    float eps, float grad_scale, int* step, void* stream) {
  if (!w || !g || !m || !v || !step) return SNNTC_E_NULL;
  if (n == 0) return SNNTC_OK;
  adam_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(w, g, m, v, n, lr, beta1, beta2, eps, grad_scale, step);
  if (done() != SNNTC_OK) return SNNTC_E_CUDA;
  step_inc_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(step);
  return done();
}

int snntc_sgdm_step(float* w, const float* g, float* vel, size_t n, float lr, float momentum, float grad_scale,
                    void* stream) {
  if (!w || !g || !vel) return SNNTC_E_NULL;
  if (n == 0) return SNNTC_OK;
  sgdm_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(w, g, vel, n, lr, momentum, grad_scale);
  return done();
}

}  // extern "C"
