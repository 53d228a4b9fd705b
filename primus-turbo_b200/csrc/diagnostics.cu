// Status reporting shared by kernels that have no status argument of their own, and a self-test of the bounded wait.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ptb {

static int *g_default_status[64] = {};
int *default_status() { return g_default_status[current_device_slot()]; }

// One CTA.  Thread 0 waits on a barrier that nobody ever arrives on, with the caller's limit: the wait must give up,
// raise the CTA's abort flag and return.  The other warps stand for the other roles of a pipelined kernel: they watch
// the abort flag (as mbar_wait does between polls) and leave when it is raised; their own watch is bounded too.  Every
// warp that saw the flag adds one to *observers; the status word receives PT_ERR_TIMEOUT.
__global__ void __launch_bounds__(128) wait_probe_kernel(uint64_t limit_ns, int *status, int *observers) {
    using namespace sm100;
    __shared__ uint64_t bar;
    __shared__ int s_abort;
    volatile int *abort_flag = &s_abort;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        ok = mbar_wait_limited(&bar, 0, abort_flag, limit_ns);
    } else {
        const uint64_t t0 = globaltimer_ns(), bound = 100 * limit_ns + 1000000ull;
        while (!*abort_flag && globaltimer_ns() - t0 < bound) __nanosleep(200);
    }
    __syncthreads();
    if (*abort_flag && (threadIdx.x & 31) == 0 && observers) atomicAdd(observers, 1);
    if (!ok && status) atomicExch(status, (int) PT_ERR_TIMEOUT);
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int pt_set_default_status(int *status) {
    g_default_status[current_device_slot()] = status;
    return PT_OK;
}

int pt_wait_probe(int64_t limit_ns, int *status, int *observers, void *stream) {
    PT_REQUIRE(limit_ns >= 1000 && limit_ns <= 1000000000ll, "wait probe: the limit must lie between 1 us and 1 s");
    PT_REQUIRE(status, "wait probe: status word required");
    wait_probe_kernel<<<1, 128, 0, (cudaStream_t) stream>>>((uint64_t) limit_ns, status, observers);
    PT_LAUNCH_OK();
    return PT_OK;
}

}  // extern "C"
