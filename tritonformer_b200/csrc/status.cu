// The library's one device-side status word (per GPU: a __device__ variable has one instance on every
// device that loads the library), its host-side reader, and a probe kernel that makes a bounded wait
// run out on purpose so that the expiry path can be tested without a fault.
#include "tc05.cuh"

namespace tfb {

__device__ int g_dev_status = 0;

// Reads (and optionally clears) the status word of the calling thread's current device.
int read_dev_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dev_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    const int z = 0;
    cudaMemcpyToSymbol(g_dev_status, &z, sizeof(int));
  }
  return v;
}

constexpr int kProbeCode = 0x7e00;

// One CTA, one warp: takes 32 columns of tensor memory like a real kernel would, then waits on an
// mbarrier that nothing ever arrives at.  The wait gives up after `limit_ns`, records kProbeCode in the
// status word, and the kernel frees its tensor memory and returns: nothing traps, nothing spins on.
__global__ void __launch_bounds__(32) wait_probe_kernel(unsigned long long limit_ns, int* waited_ok) {
  __shared__ uint64_t bar;
  __shared__ uint32_t holder;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    abort_word = 0;
  }
  __syncwarp();
  tmem_alloc(&holder, 32);
  grid_dependency_wait();
  allow_dependents();
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  const uint32_t taddr = holder;
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = mbar_wait(&bar, 0, kProbeCode, abort_flag, limit_ns);
    if (waited_ok) *waited_ok = ok ? 1 : 0;
  }
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  tmem_dealloc(taddr, 32);
}

int launch_wait_probe(unsigned long long limit_ns, int* waited_ok, cudaStream_t st) {
  wait_probe_kernel<<<1, 32, 0, st>>>(limit_ns, waited_ok);
  return launched("wait_probe");
}

}  // namespace tfb
