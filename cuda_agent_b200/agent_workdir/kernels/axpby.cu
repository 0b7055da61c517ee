// Smoke-test op of the workspace: out = alpha * a + b on fp32 vectors.
// Same launcher name and argument order as the reference's example kernel
// (agent_workdir/kernels/axpby.cu:12-20) so that its binding and model_new.py
// run unchanged; vectorised here because it costs nothing.
#include "cab_common.cuh"

namespace {

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
axpby_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
             float alpha, int size, bool vec4) {
  const int tid = blockIdx.x * THREADS + threadIdx.x;
  const int nthreads = gridDim.x * THREADS;
  int done = 0;
  if (vec4) {
    const int n4 = size >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (int i = tid; i < n4; i += nthreads) {
      const float4 x = a4[i], y = b4[i];
      o4[i] = make_float4(alpha * x.x + y.x, alpha * x.y + y.y, alpha * x.z + y.z,
                          alpha * x.w + y.w);
    }
    done = n4 << 2;
  }
  for (int i = done + tid; i < size; i += nthreads) out[i] = alpha * a[i] + b[i];
}

template <int THREADS>
int launch(float* out, const float* a, const float* b, float alpha, int size, cudaStream_t stream) {
  const bool vec4 = cab::aligned_to(out, 16) && cab::aligned_to(a, 16) && cab::aligned_to(b, 16);
  const int work = vec4 ? (size + 3) / 4 : size;
  int blocks = (work + THREADS - 1) / THREADS;
  const int cap = cab::kNumSMs * (2048 / THREADS);  // one full wave; the kernel strides
  if (blocks > cap) blocks = cap;
  axpby_kernel<THREADS><<<blocks, THREADS, 0, stream>>>(out, a, b, alpha, size, vec4);
  return cab::launch_status();
}

}  // namespace

extern "C" int axpby_launcher(float* out, const float* a, const float* b, float alpha, int size,
                              int config, cudaStream_t stream) {
  if (size <= 0) return CAB_OK;
  if (!out || !a || !b) return CAB_ERR_BAD_ARGUMENT;
  switch (config) {
    case 1: return launch<128>(out, a, b, alpha, size, stream);
    case 2: return launch<512>(out, a, b, alpha, size, stream);
    default: return launch<256>(out, a, b, alpha, size, stream);
  }
}

extern "C" const char* cab_status_string(int status) {
  switch (status) {
    case CAB_OK: return "ok";
    case CAB_ERR_BAD_ARGUMENT: return "bad argument (null pointer, non-positive or unsupported size)";
    case CAB_ERR_MISALIGNED: return "pointer not aligned as the launcher requires";
    case CAB_ERR_LAUNCH: return "CUDA reported an error for the kernel launch";
    case CAB_ERR_TOO_LARGE: return "size exceeds what this entry point supports";
    case CAB_ERR_DEVICE_STATUS: return "a kernel reported a failed bounded wait or index check";
    default: return "unknown status";
  }
}

extern "C" int cab_version(void) { return 100; }
