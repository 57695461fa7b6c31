// SnnFcGrad for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to offer at the point where the dense backward runs:
// a plugin called from inside another framework's executor that hands out only the operator's
// declared inputs and outputs, a real-time loop that fixed its memory plan up front, or a process
// whose device memory is owned by someone else's pool. The regular entry point needs a caller-owned
// workspace (u = grad/(sum w - theta) for every output, the range flag of the weight-gradient kernel
// and its partial tiles); this variant keeps that workspace inside the library image instead, as one
// fixed array in device global memory. It runs its kernels on the caller's stream only -- the
// auxiliary streams of the regular entry point are created on first use, which is an allocation.
#include "../../include/snntc_b200.h"
#include "snntc_common.cuh"

#include <limits.h>
#include <string.h>

#include <mutex>

namespace {

// The scratch lives in the library image: every GPU that loads the library holds these bytes until
// the process exits. Its NAME is only a handle on the host side; the device address must be asked
// for with cudaGetSymbolAddress (per device) before a kernel can be given it.
constexpr size_t kScratchBytes = SNNTC_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices];      // device address of g_noalloc_scratch, per device ordinal
snntc::LaunchInfo g_launch_info[kMaxDevices];
bool g_ready[kMaxDevices];

// First use on a device: resolve the array's device address and read the two device attributes the
// launch planning needs. Runs with that device current. Nothing here allocates.
int setup_current_device(int* dev_out) {
  int dev = -1;
  cudaError_t e0 = cudaGetDevice(&dev);
  if (e0 != cudaSuccess) { snntc::note_cuda_error(e0); return SNNTC_E_CUDA; }
  if (dev < 0 || dev >= kMaxDevices) return SNNTC_E_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_ready[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) { snntc::note_cuda_error(e); return SNNTC_E_CUDA; }
    int sms = 0, smem = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e != cudaSuccess) { snntc::note_cuda_error(e); return SNNTC_E_CUDA; }
    g_scratch_addr[dev] = ptr;
    g_launch_info[dev].num_sms = sms;
    g_launch_info[dev].max_smem_optin = smem;
    g_ready[dev] = true;
  }
  *dev_out = dev;
  return SNNTC_OK;
}

}  // namespace

extern "C" {

size_t snntc_noalloc_scratch_bytes(void) { return kScratchBytes; }

int snntc_fc_backward_noalloc(const float* grad_2BJ, const float* x, const float* w, const float* params6_host,
                              const float* out_2BJ, float* dx, float* dw, float* dparams6,
                              int B, int I, int w_rows, int J, void* stream) {
  if (!grad_2BJ || !x || !w || !params6_host || !out_2BJ || !dw) return SNNTC_E_NULL;
  if (B <= 0 || I <= 0 || J <= 0 || w_rows <= 0) return SNNTC_E_SHAPE;
  snntc::Geometry g;
  memset(&g, 0, sizeof(g));
  g.R = B; g.I = I; g.J = J;
  g.maxv = params6_host[0]; g.theta = params6_host[2]; g.biasvolt = params6_host[5];
  g.has_bias = g.biasvolt > 1e-8f ? 1 : 0;
  if (!(g.maxv > 1.0f)) return SNNTC_E_PARAMS;
  if (w_rows != I + g.has_bias) return SNNTC_E_WEIGHT_ROWS;
  if ((long long)B * I > INT_MAX || (long long)w_rows * J > INT_MAX || 2LL * B * J > INT_MAX) return SNNTC_E_TOO_LARGE;

  int dev = -1;
  int rc = setup_current_device(&dev);
  if (rc != SNNTC_OK) return rc;
  const snntc::LaunchInfo li = g_launch_info[dev];

  // The partial tiles of this problem must fit the fixed array; larger problems are refused, not truncated.
  const size_t need = snntc::backward_workspace_bytes(g, li);
  if (need > kScratchBytes) return SNNTC_E_WORKSPACE;

  if (dparams6) {
    const cudaError_t e = cudaMemsetAsync(dparams6, 0, 6 * sizeof(float), (cudaStream_t)stream);
    if (e != cudaSuccess) { snntc::note_cuda_error(e); return SNNTC_E_CUDA; }
  }
  // Nothing in the scratch has to start at zero: u, the flag and every partial tile the reduction reads are
  // written by this call's own kernels before they are read, whatever the previous call left there.
  snntc::Options opt;
  opt.overlap = 0;   // one stream: no auxiliary stream or event is ever created on behalf of this entry point
  rc = snntc::launch_backward(g, grad_2BJ, x, w, out_2BJ, dx, dw, g_scratch_addr[dev], kScratchBytes, li, opt,
                              (cudaStream_t)stream);
  if (rc == snntc::E_CUDA) snntc::note_cuda_error(cudaGetLastError());
  return rc;
}

}  // extern "C"
