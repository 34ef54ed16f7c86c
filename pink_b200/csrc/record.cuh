// Device helpers shared by the kernels that reduce a shard's per-neuron minima to its
// best-matching-unit record and hand the record to the other ranks.
#pragma once
#include "kernels.cuh"

namespace pinkb {

// Lexicographic order of (distance code, neuron index): lowest distance, then lowest index.
__device__ __forceinline__ bool pair_less(unsigned long long c0, unsigned long long n0,
                                          unsigned long long c1, unsigned long long n1)
{
    return c0 < c1 || (c0 == c1 && n0 < n1);
}

__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p)
{
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// First minimum of (code, local index) over keys[0..n), computed by all `threads` threads of
// the block (a multiple of 32, at most 1024).  sc/sn: one shared slot per warp.  The result is
// valid in thread 0; all threads must call.
__device__ __forceinline__ void block_argmin_keys(const unsigned long long* keys, uint32_t n, uint32_t shift,
                                                  uint32_t threads, unsigned long long* sc, unsigned long long* sn,
                                                  unsigned long long& bc, unsigned long long& bn)
{
    bc = ~0ull; bn = ~0ull;
    constexpr int kPer = 8;               // keys a thread loads per pass, all in flight at once
    for (uint32_t p0 = 0; p0 < n; p0 += threads * kPer) {
        unsigned long long k[kPer];
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const uint32_t i = p0 + e * threads + threadIdx.x;
            k[e] = i < n ? __ldcg(keys + i) : ~0ull;
        }
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const uint32_t i = p0 + e * threads + threadIdx.x;
            if (i < n && pair_less(k[e] >> shift, i, bc, bn)) { bc = k[e] >> shift; bn = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
        if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = threads >> 5;
    if (lane == 0) { sc[warp] = bc; sn[warp] = bn; }
    __syncthreads();
    if (warp == 0) {
        bc = lane < nw ? sc[lane] : ~0ull;
        bn = lane < nw ? sn[lane] : ~0ull;
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
            if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
        }
    }
}

// Hands this rank's record (code, global neuron index) to the other ranks: into pairs[rank]
// for a following all-gather, or -- peer-memory exchange -- thread r stores the two tagged words
// into rank r's record array.  Called by all threads of the block; (code, neuron) block-uniform.
__device__ __forceinline__ void publish_record(const BmuArgs& a, unsigned long long code, unsigned long long neuron)
{
    if (a.xchg_seq == 0) {
        if (threadIdx.x == 0) { a.pairs[a.rank].code = code; a.pairs[a.rank].neuron = neuron; }
        return;
    }
    if (threadIdx.x < a.world) {
        XchgRecord* rec = a.xchg_peer[threadIdx.x] + (a.xchg_seq % kXchgSlots) * a.world + a.rank;
        const unsigned long long tag = a.xchg_seq & 0xFFull;
        st_relaxed_sys(&rec->w0, (code << 8) | tag);
        st_relaxed_sys(&rec->w1, (neuron << 8) | tag);
    }
}

} // namespace pinkb
