// A kernel whose bounded wait runs out, on purpose and harmlessly: it initialises an mbarrier
// that nobody ever arrives on, waits for it with the wait that every tensor-core and bulk-copy
// kernel of this library uses (mbar_wait in blackwell.cuh) under a small iteration limit, records
// its code in the status word as those kernels do, and returns.  Nothing faults and nothing hangs;
// the context stays usable.  It exists so that the path from "a kernel gave up" to the error the
// engine raises can be tested end to end.
#include "blackwell.cuh"

namespace {

constexpr int WAIT_PROBE_CODE = 90;

__global__ void wait_probe_kernel(uint32_t limit, int* __restrict__ status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(smem_u32(&bar), 0, limit)) atomicExch(status, WAIT_PROBE_CODE);
}

}  // namespace

// Launches one tiny CTA that waits at most `limit` tries (1 .. 1,000,000) on a barrier that is
// never completed and then leaves code 90 in `status`.
MG_API int mg_wait_probe(int limit, int* status, void* stream) {
    MG_REQUIRE(status != nullptr, "wait probe: missing status word");
    MG_REQUIRE(limit >= 1 && limit <= 1000000, "wait probe: the limit must be 1..1000000 tries, got %d", limit);
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t)limit, status);
    MG_CHECK_LAUNCH("wait probe");
    return MG_OK;
}
