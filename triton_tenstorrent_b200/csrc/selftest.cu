// Self-test of the bounded-wait machinery the tensor-core kernels rely on: a one-warp kernel waits on
// an mbarrier that nothing ever completes, with a small cycle budget.  The wait must give up, record
// its site in the device status word and let the kernel return normally, leaving the context usable.
// Nothing here faults, traps or spins without limit.
#include "launch.h"
#include "ptx.cuh"

namespace b200k {

__global__ void __launch_bounds__(32) selftest_wait_timeout_kernel(uint32_t* status, long long budget_cycles,
                                                                    uint32_t* returned_flag) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);   // one arrival expected; nobody arrives
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  WaitCtx ctx{&abort_flag, status, budget_cycles};
  const bool ok = mbar_wait(&bar, 0, ctx, /*site=*/99);
  __syncwarp();
  if (threadIdx.x == 0) *returned_flag = ok ? 1u : 2u;   // 2: the wait gave up and the kernel carried on
}

int selftest_wait_timeout_at(uint32_t* status_words, long long budget_cycles, cudaStream_t stream) {
  if (budget_cycles <= 0 || budget_cycles > 4000000000ll)
    return set_error(B200K_ERR_INVALID_ARG, "selftest: budget must be in (0, 4e9] cycles");
  // word 0 is the status word; word 1 receives the kernel's own view of the outcome
  selftest_wait_timeout_kernel<<<1, 32, 0, stream>>>(status_words, budget_cycles, status_words + 1);
  count_launch();
  B200K_CHECK_LAUNCH("selftest_wait_timeout_kernel");
  return B200K_OK;
}

int selftest_wait_timeout(long long budget_cycles, cudaStream_t stream) {
  if (budget_cycles <= 0 || budget_cycles > 4000000000ll)
    return set_error(B200K_ERR_INVALID_ARG, "selftest: budget must be in (0, 4e9] cycles");
  const DeviceInfo* dev = current_device_info();
  if (dev == nullptr) return B200K_ERR_NO_DEVICE;
  return selftest_wait_timeout_at(dev->status_word, budget_cycles, stream);
}

}  // namespace b200k
