// Best-matching-unit reduction, neighbourhood update and mapping epilogue.
//
// The reference finds the best matching unit with a single-thread serial scan
// followed by a device-to-host read (find_best_matching_neuron_kernel,
// src/CudaLib/update_neurons.h:18-31, :64-80) and then rewrites every neuron
// (update_neurons_kernel, update_neurons.h:34-49); the next image's distance
// step converts the whole map again (copy_and_transform_kernel,
// src/CudaLib/generate_euclidean_distance_matrix.h:64-84).  Here one kernel per
// image does all of it on the device: update_pipe_kernel reduces the per-neuron
// minima to the best matching unit, derives the list of neurons to rewrite,
// streams them through shared memory, applies  w <- w - (w - r) * f  reading r
// through the quarter-turn/flip index permutation of a base rotation instead of
// from a materialised T x P array, and re-emits each rewritten neuron's
// quantised distance operand row and its sum of squares.  The difference, the
// product and the final subtraction are rounded separately (never contracted to
// FMA), as in the reference's CPU loop (src/SelfOrganizingMapLib/Trainer.h:167-179).
// bmu_kernel, worklist_kernel and update_kernel (one block per listed neuron)
// are the same steps as separate kernels, for neurons too large for the
// pipelined kernel's shared-memory stages.
#include "kernels.cuh"
#include "quant.cuh"
#include "ptx.cuh"
#include "record.cuh"

#include <algorithm>


namespace pinkb {

namespace {


constexpr int kBmuThreads = 512;

// Phase 1, one block: first minimum of (code, neuron) over this shard's keys -> this rank's record.
__global__ void __launch_bounds__(kBmuThreads)
bmu_kernel(BmuArgs a)
{
    __shared__ unsigned long long sc[32], sn[32];
    unsigned long long bc, bn;
    block_argmin_keys(a.keys, a.n, a.shift, kBmuThreads, sc, sn, bc, bn);
    __syncthreads();
    if (threadIdx.x == 0) { sc[0] = bc; sn[0] = bn == ~0ull ? ~0ull : shard_global(a.first_neuron, a.neuron_stride, bn); }
    __syncthreads();
    publish_record(a, sc[0], sn[0]);
}

constexpr int kListThreads = 256;

// Phase 2, one block per kListThreads neurons: pick the global best matching unit
// from the per-rank records, count the hit, re-arm the keys and emit the work list
// of the update (neurons with a non-zero factor, ascending).  A block finds the
// list position of its first entry by counting the non-zero factors before its
// range, so the list order does not depend on scheduling and no atomics are needed.
__global__ void __launch_bounds__(kListThreads)
worklist_kernel(BmuArgs a)
{
    __shared__ uint32_t warp_cnt[kListThreads / 32], warp_pre[kListThreads / 32];
    __shared__ uint32_t bmu_s;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        // lexicographic minimum over the per-rank records: lowest distance, then lowest neuron index
        unsigned long long bc = a.pairs[0].code, bn = a.pairs[0].neuron;
        for (uint32_t r = 1; r < a.world; ++r)
            if (pair_less(a.pairs[r].code, a.pairs[r].neuron, bc, bn)) { bc = a.pairs[r].code; bn = a.pairs[r].neuron; }
        const uint32_t bmu = (uint32_t)bn;
        bmu_s = bmu;
        if (blockIdx.x == 0 && shard_owns(a.first_neuron, a.neuron_stride, a.n, bmu)) {   // this rank owns the unit
            atomicAdd(&a.counts[bmu], 1u);
            if (a.bmu_log) *a.bmu_log = bmu;
        }
    }
    __syncthreads();
    const uint32_t bmu_row = bmu_s;
    auto fac = [&](uint32_t j) { return factor_of(a.factors, bmu_row, j, (uint32_t)shard_global(a.first_neuron, a.neuron_stride, j), a.n); };
    const uint32_t start = blockIdx.x * kListThreads, i = start + threadIdx.x;
    const float f = i < a.n ? fac(i) : 0.0f;
    const unsigned long long key = i < a.n ? a.keys[i] : 0ull;
    uint32_t pre = 0;                                   // non-zero factors before this block, counted per warp
    for (uint32_t j = threadIdx.x; j < start; j += kListThreads) pre += __popc(__ballot_sync(0xffffffffu, fac(j) != 0.0f));
    const uint32_t ballot = __ballot_sync(0xffffffffu, f != 0.0f);
    if (lane == 0) { warp_cnt[warp] = __popc(ballot); warp_pre[warp] = pre; }
    __syncthreads();
    uint32_t slot = __popc(ballot & ((1u << lane) - 1)), total = 0;
    for (uint32_t wv = 0; wv < kListThreads / 32; ++wv) {
        slot += warp_pre[wv] + (wv < warp ? warp_cnt[wv] : 0);
        total += warp_pre[wv] + warp_cnt[wv];
    }
    if (i < a.n) {
        a.keys[i] = kKeyEmpty;                          // re-arm every key for the next image's distance kernel
        if (f != 0.0f) {
            a.items[slot] = make_item(a, i, key, f);
        }
    }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
        *a.n_items = total;
        if (a.stats) { atomicAdd(a.stats, (unsigned long long)total); atomicAdd(a.stats + 1, (unsigned long long)total); }
    }
}

constexpr int kUpdThreads = 256;
constexpr int kUpdWarps = kUpdThreads / 32;
constexpr int kRowBatch = 12;         // neuron rows a thread keeps in flight (one float each)

// v / d for v * d < 2^32 with magic = floor(2^32 / d) + 1 (ranges checked on the host).
// magic == 0 encodes the divisor 1.
__device__ __forceinline__ uint32_t fast_div(uint32_t v, uint32_t magic) { return magic ? __umulhi(v, magic) : v; }
inline uint32_t div_magic(uint32_t d) { return d == 1 ? 0u : (uint32_t)((1ull << 32) / d) + 1; }

// Per neuron row (over all channels): where the row starts in the base
// rotation under the neuron's best transform, and where it lands in the
// distance operand (negative when the row lies outside the distance region).
struct RowInfo { int32_t src; int32_t kk; uint32_t span; };   // span: region columns [low 16 bits, high 16 bits) of the row

// One block per neuron of the shard.  The block looks up the best matching
// unit and its own update factor, leaves at once when the factor is zero, and
// otherwise walks the neuron in tasks of kRowBatch rows x 32 columns: a thread
// owns one column of the task, so its global address, its source position in
// the base rotation and its operand position advance by per-row constants
// taken from a small shared table, and kRowBatch loads are in flight per
// thread before anything depends on them.
template <int MODE>
__global__ void __launch_bounds__(kUpdThreads, 4)
update_kernel(Geometry g, UpdateArgs a, uint32_t stage_base, uint32_t magic_nd, uint32_t magic_blocks)
{
    extern __shared__ __align__(16) uint8_t dyn[];
    const uint32_t rows = g.C * g.nd;
    RowInfo* rowinfo = reinterpret_cast<RowInfo*>(dyn);                                  // [rows]
    uint8_t* crop_s = dyn + (((size_t)rows * sizeof(RowInfo) + 15) & ~size_t(15));       // operand row(s) being rebuilt
    const size_t crop_bytes = MODE == kModeF32 ? (size_t)g.Kp * 4 : (MODE == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    float* base_s = reinterpret_cast<float*>(crop_s + ((crop_bytes + 15) & ~size_t(15))); // [P] base rotation
    __shared__ __align__(8) uint64_t bar;
    __shared__ unsigned long long red[kUpdWarps];

    __shared__ UpdateItem item_s;
    __shared__ uint32_t live_s;
    if (threadIdx.x == 0) {
        live_s = blockIdx.x < *a.n_items;
        item_s = a.items[blockIdx.x];     // entries beyond n_items are stale but in bounds
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (!live_s) return;                  // fewer neurons to update than blocks
    const UpdateItem it = item_s;
    const uint32_t n = it.n, tq = it.tq;
    const float f = it.f;
    const int32_t ax = it.ax, ay = it.ay, a0 = it.a0;
    const float* bsrc = a.base + (size_t)tq * g.P;
    if (stage_base && threadIdx.x == 0) {
        // one bulk asynchronous copy (TMA) of the whole base rotation into shared memory
        mbar_expect_tx(&bar, g.P * 4);
        bulk_load(base_s, bsrc, g.P * 4, &bar);
    }
    const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    for (uint32_t rr = threadIdx.x; rr < rows; rr += kUpdThreads) {
        const uint32_t c = fast_div(rr, magic_nd), x = rr - c * g.nd;
        const uint32_t ci = x - g.off;                                   // unsigned wrap rejects x < off
        rowinfo[rr].src = (int32_t)(c * P1) + ax * (int32_t)x + a0;
        rowinfo[rr].kk = ci < g.ed ? (int32_t)(c * K1 + ci * g.ed) : -1;
        uint32_t span = g.ed << 16;
        if (g.circle && ci < g.ed) { const ushort2 r = g.circle[ci]; span = (uint32_t)r.x | ((uint32_t)r.y << 16); }
        rowinfo[rr].span = span;
    }
    __syncthreads();

    float* w = a.som + (size_t)n * g.Pp;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t blocks_per_col = (rows + kRowBatch - 1) / kRowBatch;
    const uint32_t ntask = ((g.nd + 31) / 32) * blocks_per_col;
    unsigned long long acc = 0;
    bool staged = false;
    for (uint32_t task = warp; task < ntask; task += kUpdWarps) {
        const uint32_t col = fast_div(task, magic_blocks), row0 = (task - col * blocks_per_col) * kRowBatch;
        const uint32_t y = col * 32 + lane;
        const bool valid = y < g.nd;
        const uint32_t cj = y - g.off;                                   // unsigned wrap rejects y < off
        const bool in_col = cj < g.ed;
        const int32_t ayy = ay * (int32_t)y;
        float* p0 = w + (size_t)row0 * g.nd + y;
        float v[kRowBatch];
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) {
            v[u] = 0.0f;
            if (valid && row0 + u < rows) v[u] = __ldcs(p0 + (size_t)u * g.nd);
        }
        if (stage_base && !staged) {
            if (!mbar_wait(&bar, 0)) return;      // bounded; cannot expire unless the copy faulted
            bsrc = base_s;
            staged = true;
        }
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) {
            if (valid && row0 + u < rows) {
                const RowInfo ri = rowinfo[row0 + u];
                const float rv = bsrc[ri.src + ayy];
                const float nv = __fsub_rn(v[u], __fmul_rn(__fsub_rn(v[u], rv), f));
                __stcs(p0 + (size_t)u * g.nd, nv);
                if (in_col && ri.kk >= 0) {
                    const uint32_t kk = (uint32_t)ri.kk + cj;
                    const float ov = (cj >= (ri.span & 0xFFFFu) && cj < (ri.span >> 16)) ? nv : 0.0f;   // zero outside a circular region
                    if (MODE == kModeU8) {
                        const uint32_t qv = quant_u8(ov);
                        crop_s[kk] = (uint8_t)qv;
                        acc += qv * qv;
                    } else if (MODE == kModeU16) {
                        const uint32_t qv = quant_u16(ov);
                        crop_s[kk] = (uint8_t)(qv >> 8);
                        crop_s[g.Kp + kk] = (uint8_t)(qv & 255);
                        acc += (unsigned long long)qv * qv;
                    } else {
                        reinterpret_cast<float*>(crop_s)[kk] = ov;
                    }
                }
            }
        }
    }
    __syncthreads();

    // Operand row(s) back to global memory, 16 bytes per store; the padding
    // beyond K stays as allocated (zero).
    const uint32_t row_bytes = MODE == kModeF32 ? g.K * 4 : g.K;
    const uint32_t stride_bytes = MODE == kModeF32 ? g.Kp * 4 : g.Kp;
    const uint32_t planes = MODE == kModeU16 ? 2 : 1;
    for (uint32_t pl = 0; pl < planes; ++pl) {
        uint8_t* dst = static_cast<uint8_t*>(pl ? a.a1 : a.a0) + (size_t)n * stride_bytes;
        const uint8_t* src = crop_s + (size_t)pl * g.Kp;
        const uint32_t vecs = row_bytes / 16;
        for (uint32_t i = threadIdx.x; i < vecs; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
        for (uint32_t i = vecs * 16 + threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
    if (MODE != kModeF32) {
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) red[warp] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long s = 0;
            for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
            if (MODE == kModeU8) static_cast<uint32_t*>(a.anorm)[n] = (uint32_t)s;
            else static_cast<unsigned long long*>(a.anorm)[n] = s;
        }
    }
}

// ---------------------------------------------------------------------------
// Persistent, TMA-pipelined update that also finds the best matching unit and
// its own work list: one block per SM.  Warp 0 is the producer: it streams a
// neuron (P floats) and the base rotation of its best transform into a
// shared-memory stage with two bulk asynchronous copies, and, once the consumer
// warps are done with a stage, writes the updated neuron and its rebuilt operand
// row(s) back with bulk stores.  Several stages are in flight, so the memory
// system always has tens of kilobytes outstanding per SM while the consumers
// compute from shared memory.
//
// Which neurons a block rewrites: the first `stages` entries are fixed (neurons
// blockIdx + i * gridDim), so the producer can start their copies at once --
// which base rotation a neuron needs follows from the neuron's own key, only
// the update factor depends on the best matching unit.  Meanwhile the consumer
// warps reduce the keys to the best matching unit (or pick it from the
// exchanged per-rank records), fetch its row of the factor table and compact
// the remaining neurons with a non-zero factor; compacted entry s goes to block
// s % gridDim, so every block gets the same number (+-1).  A fixed entry whose
// factor turns out to be zero is loaded in vain and skipped.  The block that is
// last to have read the keys re-arms them for the next image's distance kernel.
//
// The consumers first update the whole neuron (a thread owns one column of a
// block of rows; everything that does not depend on the neuron is computed once
// per kernel), then rebuild the operand row from the updated values, four
// elements per thread.  All waits are bounded.
constexpr int kPipeThreads = 1024;
constexpr int kPipeConsumerWarps = kPipeThreads / 32 - 1;
constexpr int kPipeConsumers = kPipeConsumerWarps * 32;
constexpr int kPipeMaxStages = 4;
constexpr int kPipeMaxItems = 256;    // neurons one block may own
constexpr int kPipeUnroll = 3;        // neuron rows a consumer thread processes together
constexpr int kPipeMaxTasks = 2;      // (row block, column) tasks per thread and neuron
constexpr int kPipeMaxUnits = 2;      // operand groups of four elements per thread and neuron

struct PipeParams
{
    uint32_t stages, stage_bytes, off_base, off_crop, crop_bytes;   // shared-memory layout of a stage
    uint32_t col_chunks, row_blocks, rows_per_block;                // consumer task grid per channel
    uint32_t magic_grid;                                            // multiply-high reciprocal of the grid size
    int* status;
};

// Shared-memory accesses by 32-bit shared-window address: the consumers' loops step such addresses
// with one 32-bit add per row instead of carrying 64-bit generic pointers.
__device__ __forceinline__ float lds_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void sts_f32(uint32_t addr, float v)
{
    asm volatile("st.shared.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void sts_u8(uint32_t addr, uint32_t v)
{
    asm volatile("st.shared.u8 [%0], %1;" :: "r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 1, %0;" :: "n"(kPipeConsumers) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(kPipeThreads, 1)
update_pipe_kernel(Geometry g, UpdateArgs a, PipeParams pp, BmuArgs b)
{
    extern __shared__ __align__(128) uint8_t pipe_dyn[];
    __shared__ __align__(8) uint64_t full_bar[kPipeMaxStages], done_bar[kPipeMaxStages], list_bar;
    __shared__ unsigned long long norm_s[kPipeMaxStages][kPipeConsumerWarps];   // per-warp partial sums of squares
    __shared__ UpdateItem items[kPipeMaxItems];
    __shared__ unsigned long long red_c[32], red_n[32];
    __shared__ uint32_t scan_s[32], bmu_s, last_s, m_s;
    __shared__ uint32_t chg_s[kPipeMaxStages][32];                            // per warp: did any value of the neuron change?
    __shared__ uint2 rng_s[kPipeMaxStages][32];                               // per warp: bit patterns of min |w|, max |w| of the new values

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < pp.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&done_bar[s], kPipeConsumerWarps);
        }
        mbar_init(&list_bar, 1);
        mbar_fence_init();
    }
    // operand staging starts as zeros: the padding beyond K is never written again
    for (uint32_t s = 0; s < pp.stages; ++s)
        for (uint32_t i = threadIdx.x; i < pp.crop_bytes / 4; i += kPipeThreads)
            reinterpret_cast<uint32_t*>(pipe_dyn + (size_t)s * pp.stage_bytes + pp.off_crop)[i] = 0;
    // Everything above is independent of earlier kernels; keys, map and operands are not.
    griddep_launch();
    griddep_wait();
    // fixed entries of this block; their factor is filled in once the best matching unit is known
    const uint32_t n_fixed = min(pp.stages * gridDim.x, b.n);               // neurons below this index are fixed entries
    const uint32_t m_fixed = b.n > blockIdx.x ? min(pp.stages, (b.n - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0u;
    if (threadIdx.x < m_fixed) {
        const uint32_t n = blockIdx.x + threadIdx.x * gridDim.x;
        items[threadIdx.x] = make_item(b, n, b.keys[n], 0.0f);
    }
    // A consumer thread owns four consecutive neurons of every chunk of 4 * kPipeConsumers; with a single
    // chunk (the usual case) their keys stay in registers, and with a single rank they are fetched here
    // already, so that the load overlaps the barrier below.
    constexpr uint32_t kChunk = 4 * kPipeConsumers;
    const bool one_chunk = b.n <= kChunk;
    unsigned long long kreg[4] = {~0ull, ~0ull, ~0ull, ~0ull};
    auto load_keys = [&](uint32_t i0) {
        if (i0 + 3 < b.n) {
            const ulonglong2 k01 = *reinterpret_cast<const ulonglong2*>(b.keys + i0);
            const ulonglong2 k23 = *reinterpret_cast<const ulonglong2*>(b.keys + i0 + 2);
            kreg[0] = k01.x; kreg[1] = k01.y; kreg[2] = k23.x; kreg[3] = k23.y;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) kreg[e] = i0 + e < b.n ? b.keys[i0 + e] : ~0ull;
        }
    };
    const bool keys_prefetched = warp != 0 && one_chunk && b.world == 1;
    if (keys_prefetched) load_keys(4 * (threadIdx.x - 32));
    fence_async_smem();                   // zeroed operand staging visible to later bulk stores
    __syncthreads();
    const uint32_t plane_bytes = g.P * 4;

    if (warp == 0) {
        // ------------------------------------------------------------ producer --
        // (the whole warp stays converged; lane 0 issues the asynchronous copies)
        auto issue = [&](uint32_t jx) {
            const uint32_t s = jx % pp.stages;
            uint8_t* st = pipe_dyn + (size_t)s * pp.stage_bytes;
            mbar_expect_tx(&full_bar[s], 2 * plane_bytes);
            bulk_load(st, a.som + (size_t)items[jx].n * g.Pp, plane_bytes, &full_bar[s]);
            bulk_load(st + pp.off_base, a.base + (size_t)items[jx].tq * g.P, plane_bytes, &full_bar[s]);
        };
        if (lane == 0)
            for (uint32_t jx = 0; jx < m_fixed; ++jx) issue(jx);
        // the consumers publish the rest of the list and the factors
        uint32_t M = 0;
        if (mbar_wait(&list_bar, 0)) M = m_s;
        else if (pp.status) atomicCAS(pp.status, kDevOk, kDevTimeoutUpdateProducer);
        uint32_t n_live = 0, n_rewritten = 0;
        for (uint32_t jx = 0; jx < M; ++jx) {
            const uint32_t s = jx % pp.stages, ph = (jx / pp.stages) & 1;
            if (!mbar_wait(&done_bar[s], ph)) { if (pp.status) atomicCAS(pp.status, kDevOk, kDevTimeoutUpdateProducer); break; }
            const uint32_t n = items[jx].n;
            // A neuron none of whose values changed (the factor is so small that every product
            // vanished against the value it is subtracted from) is not written back: neuron and
            // operand row in memory already hold exactly what the stage holds.
            const bool nonzero = items[jx].f != 0.0f;
            const bool live = nonzero && __any_sync(0xffffffffu, lane < kPipeConsumerWarps && chg_s[s][lane] != 0);
            n_live += nonzero; n_rewritten += live;
            uint8_t* st = pipe_dyn + (size_t)s * pp.stage_bytes;
            if (a.wrange && live) {
                const uint2 r = lane < kPipeConsumerWarps ? rng_s[s][lane] : make_uint2(0xFFFFFFFFu, 0u);
                const uint32_t lo = __reduce_min_sync(0xffffffffu, r.x), hi = __reduce_max_sync(0xffffffffu, r.y);
                if (lane == 0) a.wrange[n] = make_uint2(lo, hi);
            }
            if (MODE != kModeF32 && live) {
                unsigned long long tot = lane < kPipeConsumerWarps ? norm_s[s][lane] : 0ull;
                for (int o = 16; o > 0; o >>= 1) tot += __shfl_down_sync(0xffffffffu, tot, o);
                if (lane == 0) {
                    if (MODE == kModeU8) static_cast<uint32_t*>(a.anorm)[n] = (uint32_t)tot;
                    else static_cast<unsigned long long*>(a.anorm)[n] = tot;
                }
            }
            if (lane == 0) {
                if (live) {
                    bulk_store(a.som + (size_t)n * g.Pp, st, plane_bytes);
                    if (MODE == kModeF32) {
                        bulk_store(static_cast<float*>(a.a0) + (size_t)n * g.Kp, st + pp.off_crop, g.Kp * 4);
                    } else {
                        bulk_store(static_cast<uint8_t*>(a.a0) + (size_t)n * g.Kp, st + pp.off_crop, g.Kp);
                        if (MODE == kModeU16)
                            bulk_store(static_cast<uint8_t*>(a.a1) + (size_t)n * g.Kp, st + pp.off_crop + g.Kp, g.Kp);
                    }
                    bulk_commit();
                }
                if (jx + pp.stages < M) {
                    bulk_wait_read_all();             // the stage's stores no longer read it
                    issue(jx + pp.stages);
                }
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (b.stats) { atomicAdd(b.stats, (unsigned long long)n_live); atomicAdd(b.stats + 1, (unsigned long long)n_rewritten); }
            bulk_wait_all();
        }
    } else {
        // ----------------------------------------------------------- consumers --
        const uint32_t cwarp = warp - 1, ctid = threadIdx.x - 32;
        const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
        // Update tasks of this thread (the same for every neuron): channel c, column y, rows
        // [x0, x0 + 3 * full + tail).  Idle lanes and tasks get an empty range.
        const uint32_t tasks_per_channel = pp.col_chunks * pp.row_blocks, ntask = g.C * tasks_per_channel;
        uint32_t tk_si[kPipeMaxTasks], tk_x0[kPipeMaxTasks], tk_full[kPipeMaxTasks], tk_tail[kPipeMaxTasks];
        uint32_t tk_c[kPipeMaxTasks], tk_y[kPipeMaxTasks];
#pragma unroll
        for (int k = 0; k < kPipeMaxTasks; ++k) {
            const uint32_t task = cwarp + k * kPipeConsumerWarps;
            const uint32_t c = task / tasks_per_channel, tc = task - c * tasks_per_channel;
            const uint32_t chunk = tc / pp.row_blocks, blk = tc - chunk * pp.row_blocks;
            const uint32_t y = chunk * 32 + lane, x0 = blk * pp.rows_per_block;
            const bool live = task < ntask && y < g.nd && x0 < g.nd;
            const uint32_t nrows = live ? min(pp.rows_per_block, g.nd - x0) : 0;
            tk_c[k] = c; tk_y[k] = y; tk_x0[k] = x0;
            tk_full[k] = nrows / kPipeUnroll; tk_tail[k] = nrows - tk_full[k] * kPipeUnroll;
            tk_si[k] = c * P1 + x0 * g.nd + y;
        }
        // Operand units of this thread: within a segment of 128 consecutive operand elements, lane l
        // of a warp converts elements l, l + 32, l + 64, l + 96, so that every shared-memory read of a
        // warp touches 32 consecutive floats (no bank conflicts).  Elements beyond K read position 0
        // and are never stored.
        const uint32_t nunit = ((g.K + 127) / 128) * 32;
        uint32_t un_src[kPipeMaxUnits][4], un_dst[kPipeMaxUnits][4];
#pragma unroll
        for (int k = 0; k < kPipeMaxUnits; ++k) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t unit = ctid + k * kPipeConsumers;
                const uint32_t kk = (unit / 32) * 128 + (unit % 32) + 32 * e;
                const uint32_t c = kk / K1, rem = kk - c * K1, ci = rem / g.ed, cj = rem - ci * g.ed;
                const bool ok = unit < nunit && kk < g.K && in_region(g, ci, cj);   // outside a circular region: stays zero
                un_src[k][e] = ok ? 4 * (c * P1 + (g.off + ci) * g.nd + g.off + cj) : 0u;   // byte offset in the neuron
                un_dst[k][e] = ok ? kk : ~0u;
            }
        }
        const uint32_t nd = g.nd;

        // ---- best matching unit: first minimum of (code, neuron) over the keys.  A thread owns four
        //      consecutive neurons of every chunk of 4 * kPipeConsumers; with a single chunk (the
        //      usual case) their keys stay in registers for the compaction below.
        // neurons that provably keep every value (tiny factor against the spacing of their values) will count
        // as factor 0; their value ranges do not depend on the best matching unit and are fetched up front
        const bool can_skip = a.wrange != nullptr && a.rmax != nullptr;
        const uint32_t rmax_bits = can_skip ? *a.rmax : 0u;
        uint2 wr[4];
        auto load_ranges = [&](uint32_t i0) {
            if (i0 + 3 < b.n) {
                const uint4 r01 = *reinterpret_cast<const uint4*>(a.wrange + i0);
                const uint4 r23 = *reinterpret_cast<const uint4*>(a.wrange + i0 + 2);
                wr[0] = make_uint2(r01.x, r01.y); wr[1] = make_uint2(r01.z, r01.w);
                wr[2] = make_uint2(r23.x, r23.y); wr[3] = make_uint2(r23.z, r23.w);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) wr[e] = i0 + e < b.n ? a.wrange[i0 + e] : make_uint2(0u, 0u);
            }
        };
        if (can_skip && one_chunk) load_ranges(4 * ctid);
        unsigned long long bc = ~0ull, bn = ~0ull;
        if (b.world == 1) {
            for (uint32_t c0 = 0; c0 < b.n; c0 += kChunk) {
                const uint32_t i0 = c0 + 4 * ctid;
                if (!keys_prefetched) load_keys(i0);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const unsigned long long code = kreg[e] >> b.shift;
                    if (i0 + e < b.n && pair_less(code, i0 + e, bc, bn)) { bc = code; bn = i0 + e; }
                }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
                if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
            }
            if (lane == 0) { red_c[cwarp] = bc; red_n[cwarp] = bn; }
            consumer_sync();
        }
        if (cwarp == 0) {
            if (b.world == 1) {
                bc = lane < kPipeConsumerWarps ? red_c[lane] : ~0ull;
                bn = lane < kPipeConsumerWarps ? red_n[lane] : ~0ull;
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
                    if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
                }
                bn = shard_global(b.first_neuron, b.neuron_stride, bn);
            } else if (b.xchg_seq == 0) {
                // lexicographic minimum over the per-rank records: lowest distance, then lowest neuron index
                bc = b.pairs[0].code; bn = b.pairs[0].neuron;
                for (uint32_t r = 1; r < b.world; ++r)
                    if (pair_less(b.pairs[r].code, b.pairs[r].neuron, bc, bn)) { bc = b.pairs[r].code; bn = b.pairs[r].neuron; }
            } else {
                // the records arrive through peer stores: lane r waits (bounded) for rank r's record of this step
                const XchgRecord* slot = b.xchg_local + (b.xchg_seq % kXchgSlots) * b.world;
                const unsigned long long tag = b.xchg_seq & 0xFFull;
                bool arrived = true;
                for (uint32_t r = lane; r < b.world; r += 32) {
                    unsigned long long w0 = 0, w1 = 0;
                    bool seen = false;
                    // bounded by the wall clock: the other ranks are separate processes whose launches may
                    // lag behind by a host-side delay (file reads, first-launch module loading)
                    const unsigned long long limit = b.xchg_timeout_ns ? b.xchg_timeout_ns : 1000000000ull;
                    const unsigned long long t_start = global_timer_ns();
                    for (uint32_t spin = 0;; ++spin) {
                        w0 = ld_relaxed_sys(&slot[r].w0);
                        w1 = ld_relaxed_sys(&slot[r].w1);
                        if ((w0 & 0xFFull) == tag && (w1 & 0xFFull) == tag) { seen = true; break; }
                        if ((spin & 31u) == 31u && global_timer_ns() - t_start > limit) break;
                        __nanosleep(128);
                    }
                    // an absent neuron index (~0) lost its upper bits to the tag; restore it so it never wins
                    const unsigned long long oc = w0 >> 8, on = (w1 >> 8) == (~0ull >> 8) ? ~0ull : w1 >> 8;
                    if (seen && pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
                    arrived = arrived && seen;
                }
                arrived = __all_sync(0xffffffffu, arrived);
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
                    if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
                }
                if (!arrived) {               // a rank never delivered: report, and leave the map untouched
                    bn = ~0ull;
                    if (lane == 0 && b.status) atomicCAS(b.status, kDevOk, kDevTimeoutExchange);
                }
            }
            if (lane == 0) {
                const uint32_t bmu = (uint32_t)bn;          // ~0u: no best matching unit (exchange failed)
                bmu_s = bmu;
                if (blockIdx.x == 0 && shard_owns(b.first_neuron, b.neuron_stride, b.n, bmu)) {   // this rank owns the unit
                    atomicAdd(&b.counts[bmu], 1u);
                    if (b.bmu_log) *b.bmu_log = bmu;
                }
            }
        }
        consumer_sync();

        // ---- factors of the fixed entries; ordered compaction of the other neurons with a non-zero factor
        // With a single chunk and a single rank no key is read after this point, so the block can announce
        // that it is done with the keys now; the answer is needed only after the list has been built.
        const bool early_arrival = one_chunk && b.world == 1;
        uint32_t arrival = 0;
        if (early_arrival && ctid == 0) {
            __threadfence();
            arrival = atomicAdd(b.arrive, 1u);
        }
        const bool have_bmu = bmu_s != ~0u;
        const uint32_t bmu_row = have_bmu ? bmu_s : 0u;
        auto fac = [&](uint32_t j) { return factor_of(b.factors, bmu_row, j, (uint32_t)shard_global(b.first_neuron, b.neuron_stride, j), b.n); };
        if (ctid < m_fixed) {
            float ff = have_bmu ? fac(items[ctid].n) : 0.0f;
            if (can_skip && ff != 0.0f) {
                const uint2 r = a.wrange[items[ctid].n];
                if (cannot_change(ff, r.x, r.y, rmax_bits)) ff = 0.0f;
            }
            items[ctid].f = ff;
        }
        uint32_t total = 0;
        for (uint32_t c0 = 0; c0 < b.n; c0 += kChunk) {
            const uint32_t i0 = c0 + 4 * ctid;
            float f[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                f[e] = (have_bmu && i0 + e < b.n && i0 + e >= n_fixed) ? fac(i0 + e) : 0.0f;
            }
            if (can_skip) {
                if (!one_chunk) load_ranges(i0);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (f[e] != 0.0f && cannot_change(f[e], wr[e].x, wr[e].y, rmax_bits)) f[e] = 0.0f;
            }
            if (!one_chunk || b.world > 1) load_keys(i0);
            const uint32_t cnt = (f[0] != 0.0f) + (f[1] != 0.0f) + (f[2] != 0.0f) + (f[3] != 0.0f);
            uint32_t incl = cnt;                                   // inclusive scan over the warp's threads
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)lane >= o) incl += up;
            }
            if (lane == 31) scan_s[cwarp] = incl;
            consumer_sync();
            const uint32_t own = lane < kPipeConsumerWarps ? scan_s[lane] : 0u;
            uint32_t wincl = own;                                  // inclusive scan over the warps' totals
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, wincl, o);
                if ((int)lane >= o) wincl += up;
            }
            uint32_t slot = total + __shfl_sync(0xffffffffu, wincl - own, cwarp) + incl - cnt;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (f[e] != 0.0f) {
                    const uint32_t round = bmu_div(slot, pp.magic_grid);
                    if (slot - round * gridDim.x == blockIdx.x && pp.stages + round < (uint32_t)kPipeMaxItems)
                        items[pp.stages + round] = make_item(b, i0 + e, kreg[e], f[e]);
                    ++slot;
                }
            }
            total += __shfl_sync(0xffffffffu, wincl, 31);
            consumer_sync();
        }
        const uint32_t M = m_fixed + (total > blockIdx.x ? (total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u);
        if (ctid == 0) {
            m_s = M;
            mbar_arrive(&list_bar);           // the list is complete (ordered after all entries by the barrier above)
            // The block that is last to have read the keys re-arms them for the next image's
            // distance kernel; its consumers do so while the first neurons are still in flight.
            if (!early_arrival) {
                __threadfence();
                arrival = atomicAdd(b.arrive, 1u);
            }
            // (no fence behind the counter: the other blocks' key reads were complete before they arrived, and
            //  the reset and the re-armed keys only have to be visible to the next kernel)
            last_s = arrival == gridDim.x - 1;
            if (arrival == gridDim.x - 1) *b.arrive = 0;
        }
        consumer_sync();
        if (last_s)
            for (uint32_t i = ctid; i < b.n; i += kPipeConsumers) b.keys[i] = kKeyEmpty;
        for (uint32_t jx = 0; jx < M; ++jx) {
            const uint32_t s = jx % pp.stages, ph = (jx / pp.stages) & 1;
            if (!mbar_wait(&full_bar[s], ph)) { if (pp.status) atomicCAS(pp.status, kDevOk, kDevTimeoutUpdateConsumer); break; }
            const uint32_t som_a = smem_u32(pipe_dyn) + s * pp.stage_bytes;       // shared-window byte addresses
            const uint32_t base_a = som_a + pp.off_base, crop_a = som_a + pp.off_crop;
            const UpdateItem it = items[jx];
            const float f = it.f;
            if (f == 0.0f) {                  // a fixed entry outside the neighbourhood: nothing to do
                __syncwarp();
                if (lane == 0) mbar_arrive(&done_bar[s]);
                continue;
            }
            // -- w <- w - (w - r) * f over the whole neuron, kPipeUnroll rows per step:
            //    all loads, then the arithmetic, then the stores; no predicates in the steady loop
            bool changed = false;
            uint32_t lo_bits = 0xFFFFFFFFu, hi_bits = 0u;            // min |w|, max |w| of the new values, as bit patterns
            const uint32_t sw = nd * 4;                              // byte step of a neuron row
            const int32_t sb = it.ax * 4;                            // byte step of the base rotation per neuron row
#pragma unroll
            for (int k = 0; k < kPipeMaxTasks; ++k) {
                uint32_t aw = som_a + tk_si[k] * 4;
                uint32_t ab = base_a + 4 * (uint32_t)((int32_t)(tk_c[k] * P1) + it.ax * (int32_t)tk_x0[k] + it.a0 + it.ay * (int32_t)tk_y[k]);
                for (uint32_t i = 0; i < tk_full[k]; ++i) {
                    float w[kPipeUnroll], rv[kPipeUnroll], e[kPipeUnroll];
#pragma unroll
                    for (int u = 0; u < kPipeUnroll; ++u) { w[u] = lds_f32(aw + u * sw); rv[u] = lds_f32(ab + u * sb); }
#pragma unroll
                    for (int u = 0; u < kPipeUnroll; ++u) {
                        e[u] = __fsub_rn(w[u], __fmul_rn(__fsub_rn(w[u], rv[u]), f));
                        changed |= __float_as_uint(e[u]) != __float_as_uint(w[u]);
                        const uint32_t mag = __float_as_uint(e[u]) & 0x7FFFFFFFu;
                        lo_bits = min(lo_bits, mag); hi_bits = max(hi_bits, mag);
                    }
#pragma unroll
                    for (int u = 0; u < kPipeUnroll; ++u) sts_f32(aw + u * sw, e[u]);
                    aw += kPipeUnroll * sw; ab += kPipeUnroll * sb;
                }
                for (uint32_t i = 0; i < tk_tail[k]; ++i) {
                    const float w = lds_f32(aw);
                    const float e = __fsub_rn(w, __fmul_rn(__fsub_rn(w, lds_f32(ab)), f));
                    changed |= __float_as_uint(e) != __float_as_uint(w);
                    const uint32_t mag = __float_as_uint(e) & 0x7FFFFFFFu;
                    lo_bits = min(lo_bits, mag); hi_bits = max(hi_bits, mag);
                    sts_f32(aw, e);
                    aw += sw; ab += sb;
                }
            }
            {
                const bool warp_changed = __any_sync(0xffffffffu, changed);
                lo_bits = __reduce_min_sync(0xffffffffu, lo_bits);
                hi_bits = __reduce_max_sync(0xffffffffu, hi_bits);
                if (lane == 0) { chg_s[s][cwarp] = warp_changed; rng_s[s][cwarp] = make_uint2(lo_bits, hi_bits); }
            }
            consumer_sync();                  // whole neuron updated
            if (!__any_sync(0xffffffffu, lane < kPipeConsumerWarps && chg_s[s][lane] != 0)) {
                if (lane == 0) mbar_arrive(&done_bar[s]);    // nothing changed: operand row and sum stay as they are
                continue;
            }
            // -- operand row(s) from the updated values
            unsigned long long acc = 0;
#pragma unroll
            for (int k = 0; k < kPipeMaxUnits; ++k) {
                if (ctid + k * kPipeConsumers < nunit) {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = lds_f32(som_a + un_src[k][e]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t kk = un_dst[k][e];
                        if (kk != ~0u) {
                            if (MODE == kModeU8) {
                                const uint32_t qv = quant_u8(v[e]);
                                sts_u8(crop_a + kk, qv);
                                acc += qv * qv;
                            } else if (MODE == kModeU16) {
                                const uint32_t qv = quant_u16(v[e]);
                                sts_u8(crop_a + kk, qv >> 8);
                                sts_u8(crop_a + g.Kp + kk, qv & 255u);
                                acc += (unsigned long long)qv * qv;
                            } else {
                                sts_f32(crop_a + 4 * kk, v[e]);
                            }
                        }
                    }
                }
            }
            if (MODE != kModeF32) {
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
                if (lane == 0) norm_s[s][cwarp] = acc;
            }
            fence_async_smem();           // this thread's stage writes before the producer's bulk stores
            __syncwarp();
            if (lane == 0) mbar_arrive(&done_bar[s]);
        }
    }
}

// Reported distance (src/SelfOrganizingMapLib/Mapper.h:201-207: device float,
// then host sqrt): integer modes S / scale^2 rounded once to float.
template <int MODE>
__global__ void map_finalize_kernel(unsigned long long* __restrict__ keys, size_t count,
                                    float* __restrict__ dist, uint32_t* __restrict__ rot)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned long long key = keys[i];
        keys[i] = kKeyEmpty;
        const unsigned long long code = key >> key_shift(MODE);
        float d;
        if (MODE == kModeU8) d = (float)((double)code / 65025.0);
        else if (MODE == kModeU16) d = (float)((double)code / 4294836225.0);
        else d = __uint_as_float((uint32_t)code);
        dist[i] = sqrtf(d);
        rot[i] = (uint32_t)(key & ((1ull << key_shift(MODE)) - 1));
    }
}

template <int MODE>
cudaError_t update_classic(const Geometry& g, const UpdateArgs& a, cudaStream_t st)
{
    if ((uint64_t)g.P * g.nd >= (1ull << 32)) return cudaErrorInvalidValue;   // multiply-high division range
    const size_t crop = MODE == kModeF32 ? (size_t)g.Kp * 4 : (MODE == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    const size_t rows = (size_t)g.C * g.nd;
    const size_t fixed = ((rows * sizeof(RowInfo) + 15) & ~size_t(15)) + ((crop + 15) & ~size_t(15));
    const size_t staged = fixed + (size_t)g.P * 4;
    // The bulk copy needs a size that is a multiple of 16 bytes; otherwise (and
    // when a base rotation does not fit) the base is read through the cache.
    const uint32_t stage_base = staged <= 200 * 1024 && (g.P & 3) == 0;
    const size_t smem = stage_base ? staged : fixed;
    // Dynamic shared memory above 48 KB is an opt-in, per-device function attribute.
    static thread_local int attr_dev = -1;
    static thread_local size_t attr_bytes = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev != attr_dev || smem > attr_bytes)) {
        cudaError_t e = cudaFuncSetAttribute(update_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
        attr_bytes = smem;
    }
    const uint32_t blocks_per_col = (uint32_t)((rows + kRowBatch - 1) / kRowBatch);
    update_kernel<MODE><<<a.n, kUpdThreads, smem, st>>>(g, a, stage_base, div_magic(g.nd), div_magic(blocks_per_col));
    return cudaGetLastError();
}

int device_sm_count()
{
    static thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != dev_cached) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        dev_cached = dev;
    }
    return sms;
}

constexpr size_t kPipeBudget = 216 * 1024;   // of the 227 KB a block may use; the kernel has ~8 KB of static arrays

size_t pipe_stage_bytes(const Geometry& g)
{
    const size_t crop = g.mode == kModeF32 ? (size_t)g.Kp * 4 : (g.mode == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    const size_t plane = ((size_t)g.P * 4 + 127) & ~size_t(127);
    return 2 * plane + ((crop + 127) & ~size_t(127));
}

// The pipelined kernel needs bulk-copyable planes (16-byte multiples), at least two
// stages of {neuron, base rotation, operand rows} in shared memory, and every
// consumer thread keeps its tasks and operand units in registers.
bool pipe_eligible(const Geometry& g)
{
    if ((g.P & 3) != 0 || g.P != g.Pp || pipe_stage_bytes(g) * 2 > kPipeBudget || device_sm_count() <= 0) return false;
    const uint32_t chunks = (g.nd + 31) / 32;
    const uint32_t units = ((g.K + 127) / 128) * 32;
    return g.C * chunks <= (uint32_t)(kPipeMaxTasks * kPipeConsumerWarps) && units <= (uint32_t)(kPipeMaxUnits * kPipeConsumers);
}

template <int MODE>
cudaError_t update_dispatch(const Geometry& g, const UpdateArgs& a, const BmuArgs* fused, cudaStream_t st, int* status)
{
    if (!fused) return update_classic<MODE>(g, a, st);
    if (!pipe_eligible(g)) return cudaErrorInvalidValue;
    const size_t crop = MODE == kModeF32 ? (size_t)g.Kp * 4 : (MODE == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    const size_t plane = ((size_t)g.P * 4 + 127) & ~size_t(127);
    const size_t stage = pipe_stage_bytes(g), budget = kPipeBudget;
    const int sms = device_sm_count();
    PipeParams pp{};
    pp.stages = (uint32_t)std::min<size_t>(kPipeMaxStages, budget / stage);
    pp.stage_bytes = (uint32_t)stage;
    pp.off_base = (uint32_t)plane;
    pp.off_crop = (uint32_t)(2 * plane);
    pp.crop_bytes = (uint32_t)((crop + 127) & ~size_t(127));
    pp.col_chunks = (g.nd + 31) / 32;
    // as many row blocks as keep all consumer warps busy without exceeding the per-thread task cap
    pp.row_blocks = std::max<uint32_t>(1, kPipeConsumerWarps / (pp.col_chunks * g.C));
    pp.rows_per_block = (g.nd + pp.row_blocks - 1) / pp.row_blocks;
    pp.rows_per_block = (pp.rows_per_block + kPipeUnroll - 1) / kPipeUnroll * kPipeUnroll;   // whole unrolled steps
    pp.row_blocks = (g.nd + pp.rows_per_block - 1) / pp.rows_per_block;
    pp.status = status;
    uint32_t grid = std::min<uint32_t>(a.n, (uint32_t)sms);
    if ((a.n + grid - 1) / grid > (uint32_t)kPipeMaxItems) grid = (a.n + kPipeMaxItems - 1) / kPipeMaxItems;
    if ((uint64_t)a.n * grid >= (1ull << 32)) return cudaErrorInvalidValue;   // multiply-high division range
    pp.magic_grid = div_magic(grid);
    const size_t smem = (size_t)pp.stages * stage;
    static thread_local int attr_dev = -1;
    static thread_local size_t attr_bytes = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != attr_dev || smem > attr_bytes) {
        cudaError_t e = cudaFuncSetAttribute(update_pipe_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
        attr_bytes = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kPipeThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    // the kernel's set-up may overlap the tail of the kernel before it in the stream (it waits
    // with griddepcontrol.wait before it touches global memory)
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, update_pipe_kernel<MODE>, g, a, pp, *fused);
}

} // namespace

cudaError_t launch_bmu(const BmuArgs& a, uint32_t phase, cudaStream_t st)
{
    if (phase & 1u) bmu_kernel<<<1, kBmuThreads, 0, st>>>(a);
    if (phase & 2u) worklist_kernel<<<(a.n + kListThreads - 1) / kListThreads, kListThreads, 0, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_update(const Geometry& g, const UpdateArgs& a, cudaStream_t st, int* status)
{
    if (a.n == 0) return cudaSuccess;
    if (g.mode == kModeU8) return update_dispatch<kModeU8>(g, a, nullptr, st, status);
    if (g.mode == kModeU16) return update_dispatch<kModeU16>(g, a, nullptr, st, status);
    return update_dispatch<kModeF32>(g, a, nullptr, st, status);
}

bool update_can_fuse(const Geometry& g) { return pipe_eligible(g); }

cudaError_t launch_update_fused(const Geometry& g, const UpdateArgs& a, const BmuArgs& b, cudaStream_t st, int* status)
{
    if (a.n == 0 || !b.arrive) return cudaErrorInvalidValue;
    if (g.mode == kModeU8) return update_dispatch<kModeU8>(g, a, &b, st, status);
    if (g.mode == kModeU16) return update_dispatch<kModeU16>(g, a, &b, st, status);
    return update_dispatch<kModeF32>(g, a, &b, st, status);
}

cudaError_t launch_map_finalize(const Geometry& g, unsigned long long* keys, uint32_t n_img, uint32_t n,
                                float* dist, uint32_t* rot, cudaStream_t st)
{
    const size_t count = (size_t)n_img * n;
    if (count == 0) return cudaSuccess;
    unsigned blocks = (unsigned)((count + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    if (g.mode == kModeU8) map_finalize_kernel<kModeU8><<<blocks, 256, 0, st>>>(keys, count, dist, rot);
    else if (g.mode == kModeU16) map_finalize_kernel<kModeU16><<<blocks, 256, 0, st>>>(keys, count, dist, rot);
    else map_finalize_kernel<kModeF32><<<blocks, 256, 0, st>>>(keys, count, dist, rot);
    return cudaGetLastError();
}

} // namespace pinkb
