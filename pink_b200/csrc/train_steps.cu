// Whole training steps of a batch of images in ONE persistent kernel.
//
// The reference trains an image with a chain of launches and host round trips
//   generate_rotated_images -> generate_euclidean_distance_matrix (first + second step)
//   -> find_best_matching_neuron_kernel + device-to-host read -> update_neurons_kernel
//   (src/SelfOrganizingMapLib/Trainer.h:263-304, src/CudaLib/update_neurons.h:54-85).
// Training is strictly sequential (image i+1 sees the map image i left), so at a few microseconds
// of work per image the fixed cost of every launch decides the throughput.  Here one block per SM
// stays resident for a whole batch of images (their rotation sets are computed beforehand, they do not
// depend on the map) and walks, image by image, through
//
//   distance phase   uint8 / uint16 Gram-form contraction on the tensor cores (tcgen05.mma kind::i8,
//                    accumulators in tensor memory, operands streamed by TMA through a shared-memory
//                    ring; pairs of blocks share one M = 256 MMA where a shard has more than one
//                    neuron tile).  The epilogue keeps, per neuron, the first minimum over the
//                    transforms (64-bit atomicMin on (S << s | transform)) and, per image, the first
//                    minimum over the neurons in one 64-bit word ((S << s') | neuron): no reduction
//                    pass over the keys is needed afterwards.
//   grid barrier
//   update phase     every block reads the best-matching-unit word (several ranks: the ranks' words
//                    are exchanged through peer memory first), looks up the update factors of the
//                    neurons it owns, and streams those that can change through shared memory with
//                    bulk asynchronous copies:  w <- w - (w - r) * f  with r read through the
//                    quarter-turn / flip index permutation of a base rotation, each operation rounded
//                    separately as in the reference's CPU loop (Trainer.h:167-179); the quantised
//                    operand rows of rewritten neurons and their sums of squares are re-emitted.
//   grid barrier
//
// Ownership of neurons is static (a table built on the host, see step_assign_owners), so a block
// needs no compaction over all neurons to find its work.  The two phases use the same shared memory
// in turn.  Every wait -- on an mbarrier, on the grid barrier, on another rank -- is bounded; when one
// expires the block records a status code, raises its abort flag so that all later waits return at
// once, and runs to the common exit, which frees its tensor memory.
#include "kernels.cuh"
#include "ptx.cuh"
#include "quant.cuh"
#include "record.cuh"
#include "tensormap.cuh"

#include <algorithm>
#include <type_traits>
#include <vector>

namespace pinkb {

namespace {

constexpr uint32_t kMT = 512;                          // threads per block
constexpr uint32_t kEpiWarps = 12;                     // warps 2..13 read the accumulators (three per lane quadrant)
constexpr uint32_t kEpiThreads = kEpiWarps * 32;
constexpr uint32_t kConsWarps = kMT / 32 - 1;          // warps 1..15 update neurons; warp 0 moves the data
constexpr uint32_t kConsThreads = kConsWarps * 32;
constexpr uint32_t kBlockM = 128;                      // neurons per tile = tensor-memory lanes
constexpr uint32_t kBlockK = kOperandSliceBytes;       // bytes of K per ring stage
constexpr uint32_t kUmmaK = 32;                        // K per kind::i8 instruction
constexpr uint32_t kRingMax = 16, kUpdMax = 4;
constexpr uint32_t kMaxEntries = 64;                   // (neuron, channel) planes one block may rewrite per image
constexpr int kUnroll = 3;                             // neuron rows a consumer thread processes together
constexpr int kMaxTasks = 2;                           // (row block, column) tasks per consumer thread and plane
constexpr int kMaxUnits = 4;                           // operand groups of four elements per consumer thread and plane
constexpr uint32_t kRegionBudget = 208 * 1024;         // shared memory the two phases use in turn
constexpr unsigned long long kGridWaitNs = 2000000000ull;   // a grid barrier gives up after two seconds
constexpr uint32_t kStampWords = kStepStampWords;

template <int MODE> struct StepCfg;
template <> struct StepCfg<kModeU8>  { static constexpr uint32_t planes = 1, max_n = 256, cols = 256, word_shift = 32; };
template <> struct StepCfg<kModeU16> { static constexpr uint32_t planes = 2, max_n = 128, cols = 512, word_shift = 16; };

// One plane (channel) of one neuron to rewrite: local neuron index, base rotation, affine map from a
// neuron pixel (x, y) to that base rotation (src = ax * x + ay * y + a0 within the plane), update
// factor, channel, and whether it is the neuron's last plane.
struct Entry { uint32_t n, tq; int32_t ax, ay, a0; float f; uint32_t c, last; };

struct StepShared
{
    uint64_t full_bar[kRingMax], empty_bar[kRingMax], tmem_full, tmem_empty;   // distance phase
    uint64_t upd_full[kUpdMax], upd_done[kUpdMax];                             // update phase
    unsigned long long nb[256];                     // sums of squares of the transform tile in flight
    unsigned long long norm_s[kUpdMax][kConsWarps]; // per consumer warp: sum of squares of a rebuilt operand plane
    uint2 rng_s[kUpdMax][kConsWarps];               // per consumer warp: bit patterns of min |w|, max |w| of the new values
    uint32_t chg_s[kUpdMax][kConsWarps];            // per consumer warp: did any value change?
    Entry entries[kMaxEntries];
    uint32_t tmem_ptr, abort_flag, n_entries, pad;
};

struct StepParams { Geometry g; StepPlan plan; StepArgs a; };

__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 2, %0;" :: "n"(kConsThreads) : "memory");
}

__device__ __forceinline__ void epilogue_sync()
{
    asm volatile("bar.sync 1, %0;" :: "n"(kEpiThreads) : "memory");
}

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

// Records the first failure of the launch and makes every later wait of this block return at once.
__device__ __forceinline__ void step_fail(StepShared& sh, int* status, int code)
{
    if (status) atomicCAS(status, kDevOk, code);
    *reinterpret_cast<volatile uint32_t*>(&sh.abort_flag) = 1u;
}

__device__ __forceinline__ bool step_aborted(const StepShared& sh)
{
    return *reinterpret_cast<const volatile uint32_t*>(&sh.abort_flag) != 0u;
}

// Bounded mbarrier wait that also gives up as soon as this block, or (checked more rarely) any block
// of any rank of this launch, has failed.
__device__ __forceinline__ bool step_wait(uint64_t* bar, uint32_t parity, const StepShared& sh, const int* status)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && step_aborted(sh)) return false;
        if ((i & 1023u) == 1023u && status && ld_relaxed_gpu_s32(status) != kDevOk) return false;
    }
    return false;
}

// Barrier over all blocks of the launch (all are resident: one per SM, cooperative launch).  `target`
// is the number of arrivals since the launch began that completes it.
__device__ __forceinline__ void grid_sync(const StepArgs& a, StepShared& sh, uint32_t target)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        fence_proxy_async_all();          // this block's bulk stores to global memory are complete (waited for); order them too
        __threadfence();
        atomicAdd(&a.ctrl->bar, 1u);
        const unsigned long long t0 = global_timer_ns();
        uint32_t spins = 0;
        while (ld_acquire_gpu_u32(&a.ctrl->bar) + 1u < target) {
            if ((++spins & 63u) == 0u) {
                if (step_aborted(sh) || ld_relaxed_gpu_s32(a.status) != kDevOk) break;
                if (global_timer_ns() - t0 > kGridWaitNs) { step_fail(sh, a.status, kDevTimeoutGrid); break; }
            }
        }
        if (ld_relaxed_gpu_s32(a.status) != kDevOk) *reinterpret_cast<volatile uint32_t*>(&sh.abort_flag) = 1u;
        __threadfence();
    }
    __syncthreads();
}

// Device-timer stamps of every block (opt-in), eight words per image and block: 0 image begins, 1 the block's
// own distance tiles are reduced, 2 all blocks' are (first grid barrier passed), 3 work list built, 4 its own
// neurons are rewritten and stored, 5 all blocks' are (second grid barrier passed), 6 planes it rewrote,
// 7 distance tiles it computed, 8 first operand slice arrived (MMA thread), 9 last MMA issued, 10 accumulators
// complete (seen by an epilogue thread), 11 first neuron plane arrived (seen by a consumer thread).
__device__ __forceinline__ void stamp(const StepArgs& a, uint32_t img, uint32_t k, uint32_t thread)
{
    if (a.stamps && threadIdx.x == thread) a.stamps[((size_t)img * gridDim.x + blockIdx.x) * kStampWords + k] = global_timer_ns();
}

template <int MODE, bool PAIR>
__global__ void __launch_bounds__(kMT, 1)
train_steps_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                   const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                   const __grid_constant__ StepParams p)
{
    using Cfg = StepCfg<MODE>;
    using val_t = typename std::conditional<MODE == kModeU8, uint32_t, unsigned long long>::type;
    extern __shared__ uint8_t steps_dyn[];
    uint8_t* region = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(steps_dyn) + 1023) & ~uintptr_t(1023));
    __shared__ StepShared sh;
    const Geometry& g = p.g;
    const StepPlan& pl = p.plan;
    const StepArgs& a = p.a;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
    const uint32_t unit = PAIR ? blockIdx.x >> 1 : blockIdx.x;          // pair (or block) index in the distance phase
    const uint32_t n_units = PAIR ? gridDim.x >> 1 : gridDim.x;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRingMax; ++s) { mbar_init(&sh.full_bar[s], PAIR ? 2 : 1); mbar_init(&sh.empty_bar[s], 1); }
        mbar_init(&sh.tmem_full, 1);
        mbar_init(&sh.tmem_empty, kEpiWarps * (PAIR ? 2 : 1));
        for (uint32_t s = 0; s < kUpdMax; ++s) { mbar_init(&sh.upd_full[s], 1); mbar_init(&sh.upd_done[s], kConsWarps); }
        sh.abort_flag = 0;
        sh.n_entries = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_a0);
        tma_prefetch_desc(&map_b0);
        if (MODE == kModeU16) { tma_prefetch_desc(&map_a1); tma_prefetch_desc(&map_b1); }
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(&sh.tmem_ptr, Cfg::cols); tmem_relinquish_pair(); }
        else { tmem_alloc(&sh.tmem_ptr, Cfg::cols); tmem_relinquish(); }
    }
    tc_fence_before();
    if (PAIR) cluster_sync();             // the peer's barriers are initialised before anything arrives on them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_ptr;

    // ---- constants of the distance phase ---------------------------------------------------------
    constexpr uint32_t a_bytes = kBlockM * kBlockK;                      // per byte plane and stage
    const uint32_t b_rows = PAIR ? pl.n_tile / 2 : pl.n_tile;            // transform rows this block stages per K slice
    const uint32_t ring_stage_bytes = Cfg::planes * (a_bytes + pl.b_bytes);
    const uint32_t stage_tx = Cfg::planes * (a_bytes + b_rows * kBlockK);
    const uint32_t num_kb = g.Kp / kBlockK;
    const uint32_t n_items = pl.m_units * pl.n_tiles;                    // (neuron tile unit, transform tile) per image
    const uint32_t my_items = n_items > unit ? (n_items - unit + n_units - 1) / n_units : 0u;

    // ---- constants of the update phase (consumer threads: warps 1..15) ---------------------------
    const uint32_t cwarp = warp - 1, ctid = threadIdx.x - 32;
    const uint32_t nd = g.nd, P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    const uint32_t plane_bytes = P1 * 4;
    const uint32_t ntask = pl.col_chunks * pl.row_blocks;
    uint32_t tk_si[kMaxTasks], tk_x0[kMaxTasks], tk_y[kMaxTasks], tk_full[kMaxTasks], tk_tail[kMaxTasks];
#pragma unroll
    for (int k = 0; k < kMaxTasks; ++k) {
        const uint32_t task = cwarp + k * kConsWarps;
        const uint32_t chunk = task / pl.row_blocks, blk = task - chunk * pl.row_blocks;
        const uint32_t y = chunk * 32 + lane, x0 = blk * pl.rows_per_block;
        const bool live = warp != 0 && task < ntask && y < nd && x0 < nd;
        const uint32_t nrows = live ? min(pl.rows_per_block, nd - x0) : 0u;
        tk_y[k] = y; tk_x0[k] = x0;
        tk_full[k] = nrows / kUnroll; tk_tail[k] = nrows - tk_full[k] * kUnroll;
        tk_si[k] = x0 * nd + y;
    }
    // Operand units of this thread: within a segment of 128 consecutive operand elements of a plane,
    // lane l converts elements l, l + 32, l + 64, l + 96, so that every shared-memory read of a warp
    // touches 32 consecutive floats and every global store of a warp 32 consecutive bytes.
    const uint32_t nunit = ((K1 + 127) / 128) * 32;
    uint32_t un_src[kMaxUnits][4], un_dst[kMaxUnits][4];
#pragma unroll
    for (int k = 0; k < kMaxUnits; ++k) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t u = ctid + k * kConsThreads;
            const uint32_t kk = (u / 32) * 128 + (u % 32) + 32 * e;
            const uint32_t ci = kk / g.ed, cj = kk - ci * g.ed;
            const bool ok = warp != 0 && u < nunit && kk < K1 && in_region(g, ci, cj);    // outside a circular region: stays zero
            un_src[k][e] = ok ? 4 * ((g.off + ci) * nd + g.off + cj) : 0u;                // byte offset in the plane
            un_dst[k][e] = ok ? kk : ~0u;
        }
    }
    const bool can_skip = a.wrange != nullptr && a.rmax != nullptr;
    // the neuron lane j of warp 1 looks after in every image's work list (static ownership)
    const uint32_t own_n = (warp == 1 && lane < pl.owned_per_block) ? a.owners[(size_t)blockIdx.x * pl.owned_per_block + lane] : ~0u;
    uint32_t upd_base = 0;                // planes this block has streamed so far (stage and parity of the next one)

    for (uint32_t img = 0; img < a.n_img; ++img) {
        // =================================================================== distance phase ====
        stamp(a, img, 0, 0);
        if (warp == 0) {
            // ------------------------------------------------------ TMA producer --
            if (lane == 0) {
                fence_proxy_async_all();      // operand rows rewritten by the update phase (any block) before these loads
                uint32_t k = 0;
                for (uint32_t item = unit; item < n_items && !step_aborted(sh); item += n_units, ++k) {
                    const uint32_t mu = item % pl.m_units, nt = item / pl.m_units;
                    const int32_t m0 = (int32_t)((PAIR ? 2 * mu + pair_rank : mu) * kBlockM);
                    const int32_t brow = (int32_t)(a.b_row0 + img * g.T + nt * pl.n_tile + pair_rank * b_rows);
                    // All tiles walk K in the same order from the same slice: the tiles that share neuron rows (or
                    // transform rows) run at the same time on other SMs and then ask for the same L2 lines at about the
                    // same moment, which is cheaper for the L2 than the same requests spread in time (measured both ways).
                    for (uint32_t kb = 0; kb < num_kb; ++kb) {
                        const uint32_t it = (img * my_items + k) * num_kb + kb;
                        const uint32_t s = it % pl.ring_stages, ph = (it / pl.ring_stages) & 1;
                        if (!step_wait(&sh.empty_bar[s], ph ^ 1, sh, a.status)) { step_fail(sh, a.status, kDevTimeoutProducer); break; }
                        uint8_t* st = region + s * ring_stage_bytes;
                        const int32_t kx = (int32_t)(kb * kBlockK);
                        if (PAIR) {
                            const uint32_t bar = map_to_cta(smem_u32(&sh.full_bar[s]), 0);     // the issuing block's barrier
                            mbar_expect_tx_cluster(bar, stage_tx);
                            tma_load_2d_pair(st, &map_a0, bar, kx, m0);
                            tma_load_2d_pair(st + Cfg::planes * a_bytes, &map_b0, bar, kx, brow);
                            if (MODE == kModeU16) {
                                tma_load_2d_pair(st + a_bytes, &map_a1, bar, kx, m0);
                                tma_load_2d_pair(st + Cfg::planes * a_bytes + pl.b_bytes, &map_b1, bar, kx, brow);
                            }
                        } else {
                            mbar_expect_tx(&sh.full_bar[s], stage_tx);
                            tma_load_2d(st, &map_a0, &sh.full_bar[s], kx, m0);
                            tma_load_2d(st + Cfg::planes * a_bytes, &map_b0, &sh.full_bar[s], kx, brow);
                            if (MODE == kModeU16) {
                                tma_load_2d(st + a_bytes, &map_a1, &sh.full_bar[s], kx, m0);
                                tma_load_2d(st + Cfg::planes * a_bytes + pl.b_bytes, &map_b1, &sh.full_bar[s], kx, brow);
                            }
                        }
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // -------------------------------------------------------- MMA issuer --
            if (pair_rank == 0 && lane == 0) {
                const uint32_t idesc = make_idesc_u8(PAIR ? 2 * kBlockM : kBlockM, pl.n_tile);
                auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t acc) {
                    if (PAIR) umma_i8_pair(d, da, db, idesc, acc); else umma_i8(d, da, db, idesc, acc);
                };
                auto commit = [&](uint64_t* bar) {
                    if (PAIR) {
                        umma_commit_pair(smem_u32(bar));
                        umma_commit_pair(map_to_cta(smem_u32(bar), 1));
                    } else {
                        umma_commit(bar);
                    }
                };
                for (uint32_t k = 0; k < my_items && !step_aborted(sh); ++k) {
                    const uint32_t idn = img * my_items + k;
                    // the epilogue warps (of both blocks of a pair) are done with the previous tile's accumulators
                    if (!step_wait(&sh.tmem_empty, (idn & 1) ^ 1, sh, a.status)) { step_fail(sh, a.status, kDevTimeoutMma); break; }
                    tc_fence_after();
                    bool ok = true;
                    for (uint32_t kb = 0; kb < num_kb; ++kb) {
                        const uint32_t it = idn * num_kb + kb;
                        const uint32_t s = it % pl.ring_stages, ph = (it / pl.ring_stages) & 1;
                        if (!step_wait(&sh.full_bar[s], ph, sh, a.status)) { step_fail(sh, a.status, kDevTimeoutMma); ok = false; break; }
                        if (k == 0 && kb == 0) stamp(a, img, 8, 32);
                        tc_fence_after();
                        const uint32_t st = smem_u32(region + s * ring_stage_bytes);
                        const uint64_t a_hi = make_sw128_kmajor_desc(st);
                        const uint64_t b_hi = make_sw128_kmajor_desc(st + Cfg::planes * a_bytes);
#pragma unroll
                        for (uint32_t kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                            const uint64_t adv = (kk * kUmmaK) >> 4;      // 32 bytes along K inside the swizzled row
                            const uint32_t acc = (kb | kk) != 0;
                            if (MODE == kModeU8) {
                                mma(tmem_base, a_hi + adv, b_hi + adv, acc);
                            } else {
                                const uint64_t a_lo = make_sw128_kmajor_desc(st + a_bytes);
                                const uint64_t b_lo = make_sw128_kmajor_desc(st + Cfg::planes * a_bytes + pl.b_bytes);
                                mma(tmem_base, a_hi + adv, b_hi + adv, acc);                         // hh
                                mma(tmem_base + Cfg::max_n, a_lo + adv, b_lo + adv, acc);            // ll
                                mma(tmem_base + 2 * Cfg::max_n, a_hi + adv, b_lo + adv, acc);        // cross
                                mma(tmem_base + 2 * Cfg::max_n, a_lo + adv, b_hi + adv, 1u);
                            }
                        }
                        commit(&sh.empty_bar[s]);        // frees the stage once these MMAs have read it
                    }
                    if (!ok) break;
                    commit(&sh.tmem_full);               // accumulators of this tile complete
                    stamp(a, img, 9, 32);
                }
            }
            __syncwarp();
        } else if (warp < 2 + kEpiWarps) {
            // ----------------------------------------------------------- epilogue --
            // Three warps share a lane quadrant of the tensor memory and split the tile's columns; a thread
            // owns one neuron row of its third: S = |a|^2 + |b|^2 - 2ab per column, first minimum, one
            // atomicMin per row into the per-neuron key, one per warp into the image's unit word.
            val_t* nbv = reinterpret_cast<val_t*>(sh.nb);
            const uint32_t et = threadIdx.x - 64;
            const uint32_t quad = warp & 3, part = (warp - 2) >> 2;          // part 0..2 of the tile's columns
            const uint32_t row = quad * 32 + lane;
            const uint32_t chunks = pl.n_tile / 16;
            const uint32_t c_lo = (chunks * part / 3) * 16, c_hi_tile = (chunks * (part + 1) / 3) * 16;
            const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16);
            uint32_t k = 0;
            for (uint32_t item = unit; item < n_items; item += n_units, ++k) {
                const uint32_t idn = img * my_items + k;
                const uint32_t mu = item % pl.m_units, nt = item / pl.m_units;
                const uint32_t n = (PAIR ? 2 * mu + pair_rank : mu) * kBlockM + row;
                const uint32_t t0 = nt * pl.n_tile;
                const uint32_t ncols = g.T > t0 ? min(pl.n_tile, g.T - t0) : 0u;
                const size_t brow = (size_t)a.b_row0 + (size_t)img * g.T + t0;
                for (uint32_t j = et; j < pl.n_tile; j += kEpiThreads)
                    nbv[j] = j < ncols ? static_cast<const val_t*>(a.bnorm)[brow + j] : val_t(0);
                const val_t na = n < a.n ? __ldcg(static_cast<const val_t*>(a.anorm) + n) : val_t(0);
                epilogue_sync();                          // nbv visible to all epilogue warps
                const uint32_t c_hi = min(c_hi_tile, ncols);
                // Per column only the part of S that depends on it is formed, D = |b|^2 - 2ab (uint8: exact as a signed
                // 32-bit value, because S = |a|^2 + D and |a|^2 both lie in [0, 2^31)); |a|^2 is added to the winner.
                using cmp_t = typename std::conditional<MODE == kModeU8, int32_t, long long>::type;
                constexpr cmp_t kNever = MODE == kModeU8 ? (cmp_t)0x7FFFFFFF : (cmp_t)0x7FFFFFFFFFFFFFFFll;
                constexpr int kChains = 4;
                cmp_t best[kChains];
                uint32_t bcol[kChains];
#pragma unroll
                for (int c = 0; c < kChains; ++c) { best[c] = kNever; bcol[c] = 0; }
                const bool ready = step_wait(&sh.tmem_full, idn & 1, sh, a.status);
                if (ready) {
                    stamp(a, img, 10, 64);
                    tc_fence_after();
                    auto reduce = [&](uint32_t c0, const uint32_t (&x0)[16], const uint32_t (&x1)[16], const uint32_t (&x2)[16]) {
                        cmp_t sv[16];
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j) {
                            if (MODE == kModeU8) {
                                sv[j] = (cmp_t)(int32_t)((uint32_t)nbv[c0 + j] - 2u * x0[j]);
                            } else {
                                const unsigned long long dot = ((unsigned long long)x0[j] << 16)
                                                             + ((unsigned long long)x2[j] << 8) + x1[j];
                                sv[j] = (cmp_t)((unsigned long long)nbv[c0 + j] - 2ull * dot);
                            }
                        }
                        if (c0 + 16 > c_hi) {                     // ragged last chunk: columns beyond T never win
#pragma unroll
                            for (uint32_t j = 0; j < 16; ++j) if (c0 + j >= c_hi) sv[j] = kNever;
                        }
#pragma unroll
                        for (uint32_t j = 0; j < 16; ++j)
                            if (sv[j] < best[j % kChains]) { best[j % kChains] = sv[j]; bcol[j % kChains] = c0 + j; }
                    };
                    if (MODE == kModeU8) {
                        // the next chunk's tcgen05.ld is in flight while the current one is reduced
                        uint32_t xa[16], xb[16];
                        if (c_lo < c_hi) tmem_ld_32x16(lane_addr + c_lo, xa);
                        for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 32) {
                            tmem_ld_wait_on(xa);
                            if (c0 + 16 < c_hi) tmem_ld_32x16(lane_addr + c0 + 16, xb);
                            reduce(c0, xa, xa, xa);
                            if (c0 + 16 < c_hi) {
                                tmem_ld_wait_on(xb);
                                if (c0 + 32 < c_hi) tmem_ld_32x16(lane_addr + c0 + 32, xa);
                                reduce(c0 + 16, xb, xb, xb);
                            }
                        }
                    } else {
                        uint32_t x0[16], x1[16], x2[16];
                        for (uint32_t c0 = c_lo; c0 < c_hi; c0 += 16) {
                            tmem_ld_32x16(lane_addr + c0, x0);
                            tmem_ld_32x16(lane_addr + Cfg::max_n + c0, x1);
                            tmem_ld_32x16(lane_addr + 2 * Cfg::max_n + c0, x2);
                            tmem_ld_wait_on(x0); tmem_ld_wait_on(x1); tmem_ld_wait_on(x2);
                            reduce(c0, x0, x1, x2);
                        }
                    }
                } else {
                    step_fail(sh, a.status, kDevTimeoutEpilogue);
                }
                // first minimum over the chains: lowest value, then lowest column
                cmp_t best_d = best[0];
                uint32_t best_c = bcol[0];
#pragma unroll
                for (int c = 1; c < kChains; ++c)
                    if (best[c] < best_d || (best[c] == best_d && bcol[c] < best_c)) { best_d = best[c]; best_c = bcol[c]; }
                unsigned long long cand = ~0ull;              // (S, global neuron) of this row, ordered like the unit word
                if (n < a.n && ready && c_lo < c_hi) {
                    const val_t best_s = (val_t)(na + (val_t)best_d);
                    atomicMin(&a.keys[n], ((unsigned long long)best_s << key_shift(MODE)) | (unsigned long long)(t0 + best_c));
                    cand = ((unsigned long long)best_s << Cfg::word_shift) | shard_global(a.first_neuron, a.neuron_stride, n);
                }
                for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_down_sync(0xffffffffu, cand, o));
                if (lane == 0 && cand != ~0ull) atomicMin(&a.ctrl->bmu_word[img], cand);
                // hand the accumulators back to the MMA issuer (of the pair) and the column sums to the next tile
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&sh.tmem_empty), 0));
                    else mbar_arrive(&sh.tmem_empty);
                }
                epilogue_sync();
            }
        }
        stamp(a, img, 1, 64);
        grid_sync(a, sh, (2 * img + 1) * gridDim.x);
        stamp(a, img, 2, 0);

        // ===================================================================== update phase ====
        if (warp == 1) {
            const uint32_t rmax_bits = can_skip ? a.rmax[img] : 0u;
            // ---- best matching unit: the image's word, or the first minimum over the ranks' words
            const unsigned long long word = __ldcg(&a.ctrl->bmu_word[img]);
            unsigned long long bc = word == ~0ull ? ~0ull : word >> Cfg::word_shift;
            unsigned long long bn = word == ~0ull ? ~0ull : word & ((1ull << Cfg::word_shift) - 1);
            if (a.world > 1) {
                const unsigned long long seq = a.xchg_seq0 + img, tag = seq & 0xFFull;
                if (blockIdx.x == 0 && lane < a.world) {
                    // this rank's record goes into every rank's ring with two plain 8-byte stores over NVLink
                    XchgRecord* rec = a.xchg_peer[lane] + (seq % kXchgSlots) * a.world + a.rank;
                    st_relaxed_sys(&rec->w0, (bc << 8) | tag);
                    st_relaxed_sys(&rec->w1, (bn << 8) | tag);
                }
                // lane r waits (bounded by the wall clock) for rank r's record of this image
                const XchgRecord* slot = a.xchg_local + (seq % kXchgSlots) * a.world;
                bc = ~0ull; bn = ~0ull;
                bool arrived = true;
                for (uint32_t r = lane; r < a.world; r += 32) {
                    unsigned long long w0 = 0, w1 = 0;
                    bool seen = false;
                    const unsigned long long t0 = global_timer_ns();
                    for (uint32_t spin = 0; !seen; ++spin) {
                        w0 = ld_relaxed_sys(&slot[r].w0);
                        w1 = ld_relaxed_sys(&slot[r].w1);
                        if ((w0 & 0xFFull) == tag && (w1 & 0xFFull) == tag) { seen = true; break; }
                        if ((spin & 63u) == 63u) {
                            if (step_aborted(sh) || ld_relaxed_gpu_s32(a.status) != kDevOk) break;
                            if (global_timer_ns() - t0 > a.xchg_timeout_ns) break;
                        }
                    }
                    // an absent neuron index (~0) lost its upper bits to the tag; restore it so it never wins
                    const unsigned long long oc = w0 >> 8, on = (w1 >> 8) == (~0ull >> 8) ? ~0ull : w1 >> 8;
                    if (seen && pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
                    arrived = arrived && seen;
                }
                arrived = __all_sync(0xffffffffu, arrived);
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long oc = __shfl_xor_sync(0xffffffffu, bc, o), on = __shfl_xor_sync(0xffffffffu, bn, o);
                    if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
                }
                if (!arrived) {               // a rank never delivered: report, and leave the map untouched
                    bn = ~0ull;
                    if (lane == 0) step_fail(sh, a.status, kDevTimeoutExchange);
                }
            }
            const uint32_t bmu = (uint32_t)bn;              // ~0u: no best matching unit
            const bool have_bmu = bn != ~0ull && !step_aborted(sh);
            if (blockIdx.x == 0 && lane == 0) {
                if (have_bmu && shard_owns(a.first_neuron, a.neuron_stride, a.n, bmu)) {    // this rank owns the unit
                    atomicAdd(&a.counts[bmu], 1u);
                    if (a.bmu_log) a.bmu_log[img] = bmu;
                }
            }
            // ---- work list: the neurons this block owns whose factor is not zero and whose values can change
            const uint32_t n = own_n;
            const bool valid = n < a.n;
            float f = 0.0f;
            unsigned long long key = 0;
            if (valid) {
                // three independent loads (one memory round trip)
                key = __ldcg(&a.keys[n]);
                const uint2 r = can_skip ? __ldcg(&a.wrange[n]) : make_uint2(0u, 0u);
                if (have_bmu) f = factor_of(a.factors, bmu, n, (uint32_t)shard_global(a.first_neuron, a.neuron_stride, n), a.n);
                a.keys[n] = kKeyEmpty;                       // re-armed for the next image's distance phase
                if (can_skip && f != 0.0f && cannot_change(f, r.x, r.y, rmax_bits)) f = 0.0f;
            }
            const uint32_t ballot = __ballot_sync(0xffffffffu, f != 0.0f);
            if (f != 0.0f) {
                const uint32_t t = (uint32_t)(key & ((1ull << key_shift(MODE)) - 1));
                const uint32_t fl = t / g.R, r = t - fl * g.R;
                const uint32_t jq = g.q ? r / g.q : 0u;
                const int32_t ndi = (int32_t)nd, nd1 = ndi - 1, sgn = fl ? -1 : 1;
                Entry e;
                e.n = n; e.tq = g.q ? r - jq * g.q : 0u; e.f = f;
                switch (jq) {
                    case 0:  e.ax = sgn * ndi;  e.ay = 1;    e.a0 = fl ? nd1 * ndi : 0; break;
                    case 1:  e.ax = sgn;        e.ay = -ndi; e.a0 = nd1 * ndi + (fl ? nd1 : 0); break;
                    case 2:  e.ax = -sgn * ndi; e.ay = -1;   e.a0 = fl ? nd1 : nd1 * ndi + nd1; break;
                    default: e.ax = -sgn;       e.ay = ndi;  e.a0 = fl ? 0 : nd1; break;
                }
                const uint32_t pos = __popc(ballot & ((1u << lane) - 1u)) * g.C;
                for (uint32_t c = 0; c < g.C; ++c) {
                    e.c = c; e.last = c + 1 == g.C;
                    sh.entries[pos + c] = e;
                }
            }
            if (lane == 0) sh.n_entries = __popc(ballot) * g.C;
        }
        __syncthreads();
        stamp(a, img, 3, 0);
        const uint32_t M = sh.n_entries;
        const float* base_img = a.base + (size_t)img * (g.q ? g.q : 1) * g.P;

        if (warp == 0) {
            // ------------------------------------------------------------ producer --
            // (the whole warp stays converged; lane 0 issues the asynchronous copies)
            auto issue = [&](uint32_t jx) {
                const uint32_t s = (upd_base + jx) % pl.upd_stages;
                uint8_t* st = region + (size_t)s * pl.upd_stage_bytes;
                const Entry& e = sh.entries[jx];
                mbar_expect_tx(&sh.upd_full[s], 2 * plane_bytes);
                bulk_load(st, a.som + (size_t)e.n * g.Pp + (size_t)e.c * P1, plane_bytes, &sh.upd_full[s]);
                bulk_load(st + pl.upd_off_base, base_img + ((size_t)e.tq * g.C + e.c) * P1, plane_bytes, &sh.upd_full[s]);
            };
            if (lane == 0)
                for (uint32_t jx = 0; jx < M && jx < pl.upd_stages; ++jx) issue(jx);
            uint32_t n_live = 0, n_rewritten = 0;
            bool neuron_changed = false;
            uint32_t lo = 0xFFFFFFFFu, hi = 0u;
            unsigned long long tot = 0;
            for (uint32_t jx = 0; jx < M; ++jx) {
                const uint32_t gx = upd_base + jx, s = gx % pl.upd_stages, ph = (gx / pl.upd_stages) & 1;
                if (!step_wait(&sh.upd_done[s], ph, sh, a.status)) { step_fail(sh, a.status, kDevTimeoutUpdateProducer); break; }
                const Entry e = sh.entries[jx];
                // A plane none of whose values changed (the factor is so small that every product vanished
                // against the value it is subtracted from) is not written back.
                const bool changed = __any_sync(0xffffffffu, lane < kConsWarps && sh.chg_s[s][lane] != 0);
                neuron_changed = neuron_changed || changed;
                {
                    const uint2 r = lane < kConsWarps ? sh.rng_s[s][lane] : make_uint2(0xFFFFFFFFu, 0u);
                    lo = min(lo, __reduce_min_sync(0xffffffffu, r.x));
                    hi = max(hi, __reduce_max_sync(0xffffffffu, r.y));
                }
                if (changed || g.C > 1) {
                    unsigned long long part = lane < kConsWarps ? sh.norm_s[s][lane] : 0ull;
                    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                    tot += part;
                }
                uint8_t* st = region + (size_t)s * pl.upd_stage_bytes;
                if (lane == 0) {
                    if (changed) {
                        bulk_store(a.som + (size_t)e.n * g.Pp + (size_t)e.c * P1, st, plane_bytes);
                        bulk_commit();
                    }
                    if (e.last && neuron_changed) {
                        if (a.wrange) a.wrange[e.n] = make_uint2(lo, hi);
                        if (MODE == kModeU8) static_cast<uint32_t*>(a.anorm)[e.n] = (uint32_t)tot;
                        else static_cast<unsigned long long*>(a.anorm)[e.n] = tot;
                    }
                    if (jx + pl.upd_stages < M) {
                        bulk_wait_read_all();             // the stage's store no longer reads it
                        issue(jx + pl.upd_stages);
                    }
                }
                if (e.last) {
                    n_live += 1; n_rewritten += neuron_changed;
                    neuron_changed = false; lo = 0xFFFFFFFFu; hi = 0u; tot = 0;
                }
                __syncwarp();
            }
            if (lane == 0) {
                if (a.stats && n_live) { atomicAdd(a.stats, (unsigned long long)n_live); atomicAdd(a.stats + 1, (unsigned long long)n_rewritten); }
                bulk_wait_all();
            }
            __syncwarp();
        } else {
            // ----------------------------------------------------------- consumers --
            for (uint32_t jx = 0; jx < M; ++jx) {
                const uint32_t gx = upd_base + jx, s = gx % pl.upd_stages, ph = (gx / pl.upd_stages) & 1;
                // (no early exit on a failed wait: every consumer warp must reach the barriers below the same
                //  number of times; after a failure all later waits return at once and the results are void anyway)
                if (!step_wait(&sh.upd_full[s], ph, sh, a.status)) step_fail(sh, a.status, kDevTimeoutUpdateConsumer);
                if (jx == 0) stamp(a, img, 11, 32);
                const uint32_t som_a = smem_u32(region) + s * pl.upd_stage_bytes;        // shared-window byte addresses
                const uint32_t base_a = som_a + pl.upd_off_base;
                const Entry e = sh.entries[jx];
                const float f = e.f;
                // -- w <- w - (w - r) * f over the whole plane, kUnroll rows per step:
                //    all loads, then the arithmetic, then the stores; no predicates in the steady loop
                // What is tracked per element costs issue slots (the loop is issue-bound): one LOP3 for "did any bit
                // change", two integer min / max for the value range.  The range is taken over the bit patterns as
                // SIGNED integers: for non-negative floats that is the order of the values; a negative value (or
                // NaN) shows as a negative minimum, and the neuron then simply gets no "cannot change" guarantee.
                uint32_t diff_bits = 0;
                int32_t lo_i = 0x7FFFFFFF, hi_i = (int32_t)0x80000000;
                const uint32_t sw = nd * 4;                             // byte step of a neuron row
                const int32_t sb = e.ax * 4;                            // byte step of the base rotation per neuron row
#pragma unroll
                for (int k = 0; k < kMaxTasks; ++k) {
                    uint32_t aw = som_a + tk_si[k] * 4;
                    uint32_t ab = base_a + 4 * (uint32_t)(e.ax * (int32_t)tk_x0[k] + e.a0 + e.ay * (int32_t)tk_y[k]);
                    for (uint32_t i = 0; i < tk_full[k]; ++i) {
                        float w[kUnroll], rv[kUnroll], o[kUnroll];
#pragma unroll
                        for (int u = 0; u < kUnroll; ++u) { w[u] = lds_f32(aw + u * sw); rv[u] = lds_f32(ab + u * sb); }
#pragma unroll
                        for (int u = 0; u < kUnroll; ++u) {
                            o[u] = __fsub_rn(w[u], __fmul_rn(__fsub_rn(w[u], rv[u]), f));
                            diff_bits |= __float_as_uint(o[u]) ^ __float_as_uint(w[u]);
                            lo_i = min(lo_i, __float_as_int(o[u])); hi_i = max(hi_i, __float_as_int(o[u]));
                        }
#pragma unroll
                        for (int u = 0; u < kUnroll; ++u) sts_f32(aw + u * sw, o[u]);
                        aw += kUnroll * sw; ab += kUnroll * sb;
                    }
                    for (uint32_t i = 0; i < tk_tail[k]; ++i) {
                        const float w = lds_f32(aw);
                        const float o = __fsub_rn(w, __fmul_rn(__fsub_rn(w, lds_f32(ab)), f));
                        diff_bits |= __float_as_uint(o) ^ __float_as_uint(w);
                        lo_i = min(lo_i, __float_as_int(o)); hi_i = max(hi_i, __float_as_int(o));
                        sts_f32(aw, o);
                        aw += sw; ab += sb;
                    }
                }
                // this thread's stores into the stage before the producer's bulk store reads it (asynchronous proxy);
                // issued here so that its latency overlaps the barrier and the operand pass below, which only read
                if (diff_bits != 0u) fence_async_smem();
                {
                    const bool warp_changed = __any_sync(0xffffffffu, diff_bits != 0u);
                    lo_i = __reduce_min_sync(0xffffffffu, lo_i);
                    hi_i = __reduce_max_sync(0xffffffffu, hi_i);
                    // (idle warps keep the neutral range: minimum 0x7FFFFFFF, maximum below zero -> shown as 0)
                    const uint32_t lo_bits = lo_i < 0 ? 0u : (uint32_t)lo_i;
                    const uint32_t hi_bits = lo_i < 0 ? 0xFFFFFFFFu : (hi_i < 0 ? 0u : (uint32_t)hi_i);
                    if (lane == 0) { sh.chg_s[s][cwarp] = warp_changed; sh.rng_s[s][cwarp] = make_uint2(lo_bits, hi_bits); }
                }
                consumer_sync();                  // whole plane updated, flags of all warps written
                const bool plane_changed = __any_sync(0xffffffffu, lane < kConsWarps && sh.chg_s[s][lane] != 0);
                if (plane_changed || g.C > 1) {
                    // -- operand bytes of this plane from the updated values, straight to global memory, and their
                    //    sum of squares (an unchanged plane of a multi-channel neuron still contributes its sum)
                    unsigned long long acc = 0;
                    uint8_t* row0 = static_cast<uint8_t*>(a.a0) + (size_t)e.n * g.Kp + (size_t)e.c * K1;
                    uint8_t* row1 = MODE == kModeU16 ? static_cast<uint8_t*>(a.a1) + (size_t)e.n * g.Kp + (size_t)e.c * K1 : nullptr;
#pragma unroll
                    for (int k = 0; k < kMaxUnits; ++k) {
                        if (ctid + k * kConsThreads < nunit) {
                            float v[4];
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) v[q4] = lds_f32(som_a + un_src[k][q4]);
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const uint32_t kk = un_dst[k][q4];
                                if (kk != ~0u) {
                                    if (MODE == kModeU8) {
                                        const uint32_t qv = quant_u8(v[q4]);
                                        if (plane_changed) row0[kk] = (uint8_t)qv;
                                        acc += qv * qv;
                                    } else {
                                        const uint32_t qv = quant_u16(v[q4]);
                                        if (plane_changed) { row0[kk] = (uint8_t)(qv >> 8); row1[kk] = (uint8_t)(qv & 255u); }
                                        acc += (unsigned long long)qv * qv;
                                    }
                                }
                            }
                        }
                    }
                    if (MODE == kModeU8) {
                        // at most 16 squares below 2^16 per thread: the warp's sum fits 32 bits, one reduction instruction
                        const uint32_t wsum = __reduce_add_sync(0xffffffffu, (uint32_t)acc);
                        if (lane == 0) sh.norm_s[s][cwarp] = wsum;
                    } else {
                        for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
                        if (lane == 0) sh.norm_s[s][cwarp] = acc;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.upd_done[s]);
            }
        }
        upd_base += M;
        stamp(a, img, 4, 0);
        if (a.stamps && threadIdx.x == 1) {
            a.stamps[((size_t)img * gridDim.x + blockIdx.x) * kStampWords + 6] = M;
            a.stamps[((size_t)img * gridDim.x + blockIdx.x) * kStampWords + 7] = my_items;
        }
        grid_sync(a, sh, (2 * img + 2) * gridDim.x);
        stamp(a, img, 5, 0);
    }

    tc_fence_before();
    if (PAIR) cluster_sync();             // neither block leaves while the other may still signal or read it
    else __syncthreads();
    if (warp == 1) {
        if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::cols); else tmem_dealloc(tmem_base, Cfg::cols);
    }
}

template <int MODE, bool PAIR>
const void* kernel_ptr() { return reinterpret_cast<const void*>(&train_steps_kernel<MODE, PAIR>); }

const void* kernel_for(int mode, bool pair)
{
    if (mode == kModeU8) return pair ? kernel_ptr<kModeU8, true>() : kernel_ptr<kModeU8, false>();
    return pair ? kernel_ptr<kModeU16, true>() : kernel_ptr<kModeU16, false>();
}

uint32_t round_up_u32(uint32_t v, uint32_t m) { return (v + m - 1) / m * m; }

} // namespace

bool step_plan(const Geometry& g, uint32_t n_local, uint32_t n_global, StepPlan* pl, const char** why_not)
{
    *pl = StepPlan{};
    const char* dummy = "";
    if (!why_not) why_not = &dummy;
    if (g.mode != kModeU8 && g.mode != kModeU16) { *why_not = "float distances"; return false; }
    const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    if ((P1 & 3u) != 0 || g.P != g.Pp) { *why_not = "neuron planes are not a multiple of 16 bytes"; return false; }
    if (g.mode == kModeU16 && n_global >= 65536u) { *why_not = "more than 65535 neurons with uint16 distances"; return false; }
    if (n_local == 0) { *why_not = "empty shard"; return false; }
    const uint32_t max_n = g.mode == kModeU8 ? 256u : 128u, planes = g.mode == kModeU8 ? 1u : 2u;

    // update phase: stages of {neuron plane, base rotation plane}
    const uint32_t plane = round_up_u32(P1 * 4, 128);
    pl->upd_stage_bytes = 2 * plane;
    pl->upd_off_base = plane;
    pl->upd_stages = std::min<uint32_t>(kUpdMax, kRegionBudget / pl->upd_stage_bytes);
    if (pl->upd_stages < 2) { *why_not = "two neuron planes and two base rotation planes do not fit shared memory"; return false; }
    pl->col_chunks = (g.nd + 31) / 32;
    if (pl->col_chunks > (uint32_t)kMaxTasks * kConsWarps) { *why_not = "neuron side too large"; return false; }
    pl->row_blocks = std::max<uint32_t>(1, (uint32_t)kMaxTasks * kConsWarps / pl->col_chunks);
    pl->rows_per_block = (g.nd + pl->row_blocks - 1) / pl->row_blocks;
    pl->rows_per_block = round_up_u32(pl->rows_per_block, kUnroll);          // whole unrolled steps
    pl->row_blocks = (g.nd + pl->rows_per_block - 1) / pl->rows_per_block;
    if (((K1 + 127) / 128) * 32 > (uint32_t)kMaxUnits * kConsThreads) { *why_not = "distance region too large"; return false; }

    // how many blocks can be resident at once
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess
        || sms <= 0) { cudaGetLastError(); *why_not = "no device"; return false; }
    pl->pair = n_local > kBlockM;
    const uint32_t m_tiles = (n_local + kBlockM - 1) / kBlockM;
    pl->m_units = pl->pair ? (m_tiles + 1) / 2 : m_tiles;
    const uint32_t units_max = pl->pair ? (uint32_t)sms / 2 : (uint32_t)sms;

    // distance phase: balanced transform tiles, each a multiple of 16 columns -- the fewest tiles of at most
    // max_n columns unless that leaves blocks without a tile; then narrower tiles spread over all of them
    uint32_t tiles = (g.T + max_n - 1) / max_n;
    if ((uint64_t)pl->m_units * tiles < units_max) {
        const uint32_t most = std::max<uint32_t>(tiles, g.T / 32);
        tiles = std::max<uint32_t>(tiles, std::min<uint32_t>(most, units_max / pl->m_units));
    }
    pl->n_tile = std::min<uint32_t>(max_n, round_up_u32((g.T + tiles - 1) / tiles, 16));
    pl->n_tiles = (g.T + pl->n_tile - 1) / pl->n_tile;
    const uint32_t b_box = pl->pair ? pl->n_tile / 2 : pl->n_tile;
    pl->b_bytes = round_up_u32(b_box * kBlockK, 1024);
    const uint32_t ring_stage = planes * (kBlockM * kBlockK + pl->b_bytes);
    pl->ring_stages = std::max(2u, std::min(std::min(kRingMax, kRegionBudget / ring_stage), g.Kp / kBlockK));
    if (pl->ring_stages * ring_stage > kRegionBudget) { *why_not = "distance ring does not fit"; return false; }

    // blocks: enough for every distance tile and for one neuron each, at most one per SM
    const uint32_t items = pl->m_units * pl->n_tiles;
    uint32_t blocks = std::max<uint32_t>(items * (pl->pair ? 2u : 1u), n_local);
    blocks = std::min<uint32_t>(blocks, pl->pair ? units_max * 2 : units_max);
    if (pl->pair) blocks = std::max(2u, blocks & ~1u);
    pl->smem_bytes = std::max(pl->ring_stages * ring_stage, pl->upd_stages * pl->upd_stage_bytes) + 1024;
    {
        // ask the runtime how many of these blocks (pairs) it can really hold at once
        const void* fn = kernel_for(g.mode, pl->pair != 0);
        if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem_bytes) != cudaSuccess) {
            cudaGetLastError(); *why_not = "shared memory size refused"; return false;
        }
        if (pl->pair) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(blocks, 1, 1);
            cfg.blockDim = dim3(kMT, 1, 1);
            cfg.dynamicSmemBytes = pl->smem_bytes;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg) != cudaSuccess || clusters < 1) {
                cudaGetLastError(); *why_not = "no resident block pair"; return false;
            }
            blocks = std::min<uint32_t>(blocks, 2u * (uint32_t)clusters);
        } else {
            int per_sm = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, (int)kMT, pl->smem_bytes) != cudaSuccess || per_sm < 1) {
                cudaGetLastError(); *why_not = "no resident block"; return false;
            }
        }
    }
    pl->grid = blocks;
    pl->owned_per_block = (n_local + blocks - 1) / blocks;
    if (pl->owned_per_block > kStepMaxOwned || pl->owned_per_block * g.C > kMaxEntries) { *why_not = "too many neurons per block"; return false; }
    return true;
}

// Greedy assignment in index order: a neuron goes to the block (with room left) whose neurons so far are
// farthest from it, closeness measured by the update factors themselves -- the factor of (i, m) is large exactly when
// i and m are rewritten together.  The neighbourhood of any best matching unit then spreads over the
// blocks almost evenly (measured on a hexagonal map of 2791 neurons, sigma 3: at most 5-7 neurons of a
// block among the ~700-1000 neurons an image rewrites, against 7-9 for a round-robin assignment).
void step_assign_owners(const std::function<float(uint32_t, uint32_t)>& closeness, uint32_t first, uint32_t stride,
                        uint32_t count, const StepPlan& pl, uint32_t* owners)
{
    const uint32_t G = pl.grid, J = pl.owned_per_block;
    std::fill(owners, owners + (size_t)G * J, ~0u);
    std::vector<uint32_t> color(count), load(G, 0);
    std::vector<double> score(G);
    for (uint32_t i = 0; i < count; ++i) {
        std::fill(score.begin(), score.end(), 0.0);
        const uint32_t gi = first + i * stride;
        for (uint32_t m = 0; m < i; ++m) score[color[m]] += std::fabs((double)closeness(gi, first + m * stride));
        uint32_t best = G;
        for (uint32_t c = 0; c < G; ++c) {
            if (load[c] >= J) continue;
            if (best == G || score[c] < score[best] || (score[c] == score[best] && load[c] < load[best])) best = c;
        }
        color[i] = best;
        owners[(size_t)best * J + load[best]++] = i;
    }
}

cudaError_t launch_train_steps(const Geometry& g, const StepPlan& pl, const StepArgs& a, cudaStream_t st, const char** why)
{
    *why = "";
    if (a.n_img == 0) return cudaSuccess;
    if (a.n_img > kStepBatchMax) { *why = "too many images for one launch"; return cudaErrorInvalidValue; }
    const uint32_t b_box = pl.pair ? pl.n_tile / 2 : pl.n_tile;
    CUtensorMap ma0, ma1, mb0, mb1;
    bool ok = make_map(&ma0, a.a0, a.n, g.Kp, kBlockM) && make_map(&mb0, a.b0, a.b_rows, g.Kp, b_box);
    if (g.mode == kModeU16) ok = ok && make_map(&ma1, a.a1, a.n, g.Kp, kBlockM) && make_map(&mb1, a.b1, a.b_rows, g.Kp, b_box);
    else { ma1 = ma0; mb1 = mb0; }
    if (!ok) { *why = "cuTensorMapEncodeTiled failed"; return cudaErrorInvalidValue; }

    const void* fn = kernel_for(g.mode, pl.pair != 0);
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes);
    if (e != cudaSuccess) { *why = "cudaFuncSetAttribute(train_steps_kernel)"; return e; }

    StepParams p;
    p.g = g; p.plan = pl; p.a = a;
    void* args[5] = { &ma0, &ma1, &mb0, &mb1, &p };
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.grid, 1, 1);
    cfg.blockDim = dim3(kMT, 1, 1);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.pair ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // all blocks wait for one another at the grid barriers: the launch must place them all at once
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.plain_launch ? 1 : 2;       // without the attribute the caller vouches for an otherwise idle device
    *why = "train_steps_kernel launch";
    return cudaLaunchKernelExC(&cfg, fn, args);
}

} // namespace pinkb
