// Self-test of the bounded device waits that every tcgen05 kernel in this library is built on.
//
// The kernels never spin without a limit: a wait that runs out records where it gave up in a status word, raises
// the CTA's abort flag and returns, so the kernel drains and exits with the context intact. That path cannot be
// reached by a healthy launch, so this file gives it a launch of its own: one warp waits, with a short limit, on
// a barrier that nothing ever arrives on, gives up, and the kernel ends normally. The host then reads the record.
// No trap, no fault, no hang: the whole kernel runs for `limit_cycles` SM clocks plus a few microseconds.
#include "sm100_ptx.cuh"

namespace feather {
namespace selftest {

__device__ uint32_t g_status[2];

__global__ void __launch_bounds__(64, 1) wait_runs_out_kernel(long long limit_cycles, uint32_t* observed) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    const WaitGuard guard{&abort_word, g_status};
    if (threadIdx.x == 0) {
        abort_word = 0u;
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncthreads();
    bool completed = true;
    if (threadIdx.x == 0) {
        // phase 0 of a barrier that expects one arrival and gets none
        completed = guard.wait_at_most(&bar, 0u, kSiteLoadFull, 5u, limit_cycles);
    } else if (threadIdx.x == 32) {
        // a second waiter with a far longer limit: it must leave through the abort flag the first one raises
        completed = guard.wait_at_most(&bar, 0u, kSiteOperandFull, 6u, limit_cycles * 64);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        observed[0] = completed ? 1u : 0u;   // 0: the wait gave up, as it must
        observed[1] = abort_word;
    }
    if (threadIdx.x == 32) observed[2] = completed ? 1u : 0u;
}

}  // namespace selftest
}  // namespace feather

// Launches the self-test on `stream`, synchronizes it and returns what happened: out[0] = status word (wait site |
// tag << 8) the give-up recorded, out[1] = block index recorded, out[2] = 1 if the first waiter's wait "completed"
// (it must not), out[3] = the CTA's abort flag after the wait, out[4] = 1 if the second waiter "completed" (it must
// leave through the abort flag instead). `limit_cycles` is clamped to [1e5, 4e9] (at most about two seconds).
// `scratch` is device memory for three uint32 (the caller owns it; nothing is allocated here).
// Returns 0 on success, 1 if a CUDA call failed. No counterpart in the reference (its kernels have no device waits).
extern "C" int feather_selftest_wait_runs_out(long long limit_cycles, uint32_t* scratch, uint32_t* out, cudaStream_t stream) {
    using namespace feather::selftest;
    if (scratch == nullptr || out == nullptr) return 1;
    if (limit_cycles < 100000LL) limit_cycles = 100000LL;
    if (limit_cycles > 4000000000LL) limit_cycles = 4000000000LL;
    const uint32_t zero[2] = {0u, 0u};
    if (cudaMemcpyToSymbolAsync(g_status, zero, sizeof(zero), 0, cudaMemcpyHostToDevice, stream) != cudaSuccess) return 1;
    wait_runs_out_kernel<<<1, 64, 0, stream>>>(limit_cycles, scratch);
    if (cudaGetLastError() != cudaSuccess) return 1;
    uint32_t seen[3] = {9u, 9u, 9u};
    if (cudaMemcpyAsync(seen, scratch, sizeof(seen), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return 1;
    if (cudaMemcpyFromSymbolAsync(out, g_status, sizeof(zero), 0, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return 1;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return 1;
    out[2] = seen[0];
    out[3] = seen[1];
    out[4] = seen[2];
    return 0;
}
