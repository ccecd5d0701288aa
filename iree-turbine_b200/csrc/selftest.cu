// Self-test of the bounded-wait exit every kernel of this library relies on: a kernel that waits on
// a barrier nobody will ever arrive on, with a limit of a few milliseconds, and comes back the way
// the real kernels do when a wait runs out -- the shared abort word is set, every thread reaches the
// common exit, a code is OR-ed into the caller's status word, the context stays usable.  Nothing
// traps, faults or spins without a limit.
#include "common.cuh"
#include "ptx.cuh"

namespace b200k {
namespace {

__global__ void bounded_wait_selftest_kernel(int32_t* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  // warp 0 waits for a phase that never completes; warp 1 waits on the same barrier and gives up
  // as soon as it sees the abort word, as the other roles of a real kernel do
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_limit(&bar, 0, &abort_word, threadIdx.x == 0 ? limit_ns : 100ull * limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && status) {
    if (!ok && abort_word != 0) atomicOr(status, kStatusSelftestTimeout);
  }
}

}  // namespace

int launch_bounded_wait_selftest(int32_t* status, uint32_t limit_us, cudaStream_t stream) {
  if (!status) return set_error(B200K_ERR_NULL, "selftest_bounded_wait: status must be non-NULL");
  if (limit_us == 0 || limit_us > 100000)
    return set_error(B200K_ERR_BAD_SHAPE, "selftest_bounded_wait: limit_us must be in [1, 100000]");
  int rc = ensure_sm100();
  if (rc) return rc;
  bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(status, static_cast<uint64_t>(limit_us) * 1000ull);
  return check_cuda(cudaGetLastError(), "bounded_wait_selftest_kernel launch");
}

}  // namespace b200k
