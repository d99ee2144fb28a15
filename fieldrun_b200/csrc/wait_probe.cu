// A wait that is meant to run out.
//
// Every wait of the TMA-fed kernels is bounded: when a copy or a product never arrives, the waiting thread
// gives up after its limit, leaves a code in the status word and the block returns through its common exit
// (tma.cuh, bar_wait).  This entry point exercises exactly that path on purpose and harmlessly: one block
// initialises an mbarrier that nothing will ever arrive on, waits on it with a short limit, records the code
// and returns.  No copy is in flight, no tensor memory is held, nothing faults and nothing spins for ever;
// the context stays usable.  It exists so that the way from a device-side give-up to a host-side error can
// be tested.
#include "tma.cuh"

#define FRB_WAIT_PROBE_CODE 99

__global__ void wait_probe_kernel(long long limit_cycles, int* status, long long* waited_cycles) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int failed;
    if (threadIdx.x == 0) {
        failed = 0;
        frb_tma::bar_init(&bar, 1);
        frb_tma::bar_init_fence();
        const long long start = clock64();
        const bool arrived = frb_tma::bar_wait(&bar, 0, &failed, limit_cycles);   // nothing arrives: this gives up
        if (waited_cycles) *waited_cycles = clock64() - start;
        if (!arrived) atomicExch(status, FRB_WAIT_PROBE_CODE);
    }
}

// status: one int on the device (the status word the other kernels use).  limit_cycles: 1 .. 10^8 (a twentieth of
// a second at most).  waited_cycles: optional, one long long on the device.
FRB_API int frb_wait_probe(long long limit_cycles, int* status, long long* waited_cycles, cudaStream_t stream) {
    FRB_CHECK_ARG(status != nullptr, "wait_probe: no status word");
    FRB_CHECK_ARG(limit_cycles >= 1 && limit_cycles <= 100000000ll, "wait_probe: a limit of %lld cycles is outside 1..10^8",
                  limit_cycles);
    wait_probe_kernel<<<1, 32, 0, stream>>>(limit_cycles, status, waited_cycles);
    FRB_RETURN_LAUNCH("wait_probe");
}
