// Device helpers shared by the kernels that reduce a shard's per-neuron minima to its
// best-matching-unit record and hand the record to the other ranks.
#pragma once
#include "kernels.cuh"

namespace pinkb {

// Global index of local neuron j of a shard, and the inverse test: does the shard (first, stride, n) hold global neuron g?
__device__ __forceinline__ unsigned long long shard_global(uint32_t first, uint32_t stride, unsigned long long j)
{
    return first + j * stride;
}

__device__ __forceinline__ bool shard_owns(uint32_t first, uint32_t stride, uint32_t n, uint32_t g)
{
    if (g < first) return false;
    const uint32_t d = g - first;
    return d % stride == 0 && d / stride < n;
}

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

// v / d for v * d < 2^32 with magic = floor(2^32 / d) + 1; magic == 0 encodes the divisor 1.
__device__ __forceinline__ uint32_t bmu_div(uint32_t v, uint32_t magic) { return magic ? __umulhi(v, magic) : v; }

// Transform index -> base rotation and affine source map of a work-list entry.
__device__ __forceinline__ UpdateItem make_item(const BmuArgs& a, uint32_t i, unsigned long long key, float f)
{
    const uint32_t t = (uint32_t)(key & ((1ull << a.shift) - 1));
    const uint32_t fl = bmu_div(t, a.magic_R), r = t - fl * a.R;
    const uint32_t jq = a.q ? bmu_div(r, a.magic_q) : 0;
    const int32_t nd = (int32_t)a.nd, nd1 = nd - 1, sgn = fl ? -1 : 1;
    UpdateItem it;
    it.n = i;
    it.tq = a.q ? r - jq * a.q : 0;
    it.f = f;
    switch (jq) {
        case 0:  it.ax = sgn * nd;  it.ay = 1;   it.a0 = fl ? nd1 * nd : 0; break;
        case 1:  it.ax = sgn;       it.ay = -nd; it.a0 = nd1 * nd + (fl ? nd1 : 0); break;
        case 2:  it.ax = -sgn * nd; it.ay = -1;  it.a0 = fl ? nd1 : nd1 * nd + nd1; break;
        default: it.ax = -sgn;      it.ay = nd;  it.a0 = fl ? 0 : nd1; break;
    }
    return it;
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
