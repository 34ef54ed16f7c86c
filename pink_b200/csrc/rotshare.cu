// Hand-shake for rotation sets that the ranks compute in shares and copy to one another: a
// rank announces "my share of batch `seq` has arrived everywhere" by storing seq + 1 into its
// entry of a flag row in EVERY rank's memory (plain stores over NVLink, issued after the copies
// in stream order), and a rank waits -- bounded -- until all entries of the row carry that value
// before its distance kernels read the batch.  No reference counterpart (the reference trains on
// one GPU).
#include "kernels.cuh"
#include "ptx.cuh"
#include "record.cuh"

namespace pinkb {

namespace {

struct FlagPeers { unsigned long long* flags[kXchgMaxRanks]; };

__global__ void flag_publish_kernel(FlagPeers peers, uint32_t world, uint32_t entry, unsigned long long value)
{
    if (threadIdx.x < world) st_relaxed_sys(peers.flags[threadIdx.x] + entry, value);
}

__global__ void flag_wait_kernel(const unsigned long long* row, uint32_t world, uint32_t self, unsigned long long value,
                                 int* status, unsigned long long timeout_ns)
{
    bool seen = true;
    for (uint32_t r = threadIdx.x; r < world; r += 32) {
        if (r == self) continue;          // this rank's own share is ordered by its streams, never by a kernel waiting for a kernel
        bool ok = false;
        const unsigned long long t_start = global_timer_ns();       // bounded by the wall clock
        for (uint32_t spin = 0;; ++spin) {
            if (ld_relaxed_sys(row + r) == value) { ok = true; break; }
            if ((spin & 31u) == 31u && global_timer_ns() - t_start > timeout_ns) break;
            __nanosleep(128);
        }
        seen = seen && ok;
    }
    if (!__all_sync(0xffffffffu, seen) && threadIdx.x == 0 && status) atomicCAS(status, kDevOk, kDevTimeoutRotation);
    __threadfence_system();               // the copied batch is read only after the flags were seen
}

} // namespace

cudaError_t launch_flag_publish(unsigned long long* const* peer_flags, uint32_t world, uint32_t entry,
                                unsigned long long value, cudaStream_t st)
{
    if (world > kXchgMaxRanks) return cudaErrorInvalidValue;
    FlagPeers p{};
    for (uint32_t r = 0; r < world; ++r) p.flags[r] = peer_flags[r];
    flag_publish_kernel<<<1, 32, 0, st>>>(p, world, entry, value);
    return cudaGetLastError();
}

cudaError_t launch_flag_wait(const unsigned long long* row, uint32_t world, uint32_t self, unsigned long long value,
                             int* status, unsigned long long timeout_ns, cudaStream_t st)
{
    flag_wait_kernel<<<1, 32, 0, st>>>(row, world, self, value, status, timeout_ns ? timeout_ns : 1000000000ull);
    return cudaGetLastError();
}

} // namespace pinkb
