// Self-test of the bounded-wait error path every pipelined kernel of the library relies on.
//
// The kernels never spin without a limit: a role that waits on an mbarrier gives up after a cycle
// budget, records a code in the per-device error word, raises a CTA-wide flag that makes every
// later wait of the CTA return at once, and the kernel ends normally. That path cannot be
// reached through the real kernels without breaking one of them, so this file exercises the same
// helpers in the smallest possible setting: one CTA waits, with a budget of about a millisecond,
// on a barrier that nothing will ever arrive on. Nothing traps, nothing spins without a bound,
// and the context stays usable.
#include "../../include/carat_b200.h"
#include "context.cuh"
#include "ptx.cuh"

using namespace carat_b200;

namespace {

constexpr int selftest_code = 90;
constexpr long long short_limit = 2000000LL;   // about one millisecond of cycles

// report[0] = 1 when the first wait gave up, report[1] = 1 when a second wait on the same barrier
// returned without waiting again (the CTA flag was up), report[2] = cycles the second wait took.
__global__ void bounded_wait_selftest_kernel(int *device_error, int *report) {
  __shared__ __align__(8) unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbarrier_init(ptx::smem_u32(&barrier), 1);
    ptx::fence_mbarrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t bar = ptx::smem_u32(&barrier);
    const bool first = ptx::mbarrier_wait_checked(bar, 0, &abort_flag, device_error, selftest_code,
                                                  short_limit);
    const long long start = clock64();
    const bool second = ptx::mbarrier_wait_checked(bar, 0, &abort_flag, device_error,
                                                   selftest_code + 1, short_limit);
    const long long spent = clock64() - start;
    report[0] = first ? 0 : 1;
    report[1] = (!second && spent < short_limit / 4) ? 1 : 0;
    report[2] = static_cast<int>(spent < 0x7FFFFFFF ? spent : 0x7FFFFFFF);
  }
}

} // namespace

extern "C" int carat_b200_selftest_bounded_wait(int *device_report, void *stream) {
  if (device_report == nullptr) {
    set_last_error("invalid self-test report buffer");
    return -1;
  }
  int *device_error = device_error_word();
  if (device_error == nullptr) {
    set_last_error("device error word is unavailable");
    return -101;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_error,
                                                                               device_report);
  return check_cuda(cudaPeekAtLastError(), "launch bounded-wait self-test");
}
