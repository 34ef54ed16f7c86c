// Integer-mode distance kernel on the 5th-generation tensor cores.
//
// Replaces the reference's euclidean_distance_kernel + second_step_kernel
//   (src/CudaLib/euclidean_distance_kernel.h:61-102: one block per (transform,
//    neuron) pair streaming both operands;
//    src/CudaLib/generate_euclidean_distance_matrix_second_step.h:18-38: serial
//    minimum over transforms per neuron)
// by the Gram form  S[n][t] = |a_n|^2 + |b_t|^2 - 2 * a_n . b_t  where the dot
// products are a dense [n x K] x [K x T] contraction run as tcgen05.mma
// kind::i8 (u8 x u8 -> s32, accumulators in tensor memory).  All terms are
// exact integers, so S equals the reference's sum of squared differences
// bit for bit.  The epilogue reads the accumulators with tcgen05.ld, forms S,
// keeps the first minimum over the tile's transforms per neuron row and merges
// tiles with one 64-bit atomicMin per row; the N x T matrix is never written
// (unless a debug output is requested).
//
// uint16 operands are split into high and low bytes (a = 256*ah + al) and the
// dot product is assembled from three s32 accumulators
//   hh = ah.bh,  ll = al.bl,  cross = ah.bl + al.bh,
//   a.b = 65536*hh + 256*cross + ll        (combined in 64-bit integers).
//
// float32 mapping uses the same pipeline as a filter (kModeTf32): the operands are split into two TF32 words per
// value (a = ah + al with ah = the top 19 bits of a), the dot product is assembled as ah.bh + ah.bl + al.bh in
// float accumulators (kind::tf32; one for the even and one for the odd K steps), and the estimate
// |a|^2 + |b|^2 - 2 a.b of every (neuron, transform) pair is
// written out; an exact pass over the few transforms per neuron that the estimate cannot rule out follows
// (filter_f32.cu).
//
// A CTA computes a 128-neuron x n_tile-transform tile.  The kernel is bound by the operand bytes an
// SM pulls from L2, so two CTAs of a cluster work as a pair where possible (tcgen05 cta_group::2:
// one M=256 MMA over both CTAs' neuron rows; each CTA stages only half of the transform rows; the
// even CTA issues, its commits signal both CTAs).  No TMA multicast is used.  Warp 0 streams
// 128-byte-swizzled K slices of both operands with TMA into a multi-stage
// shared-memory ring, warp 1 issues the MMAs, warps 2-5 run the epilogue.
// Every mbarrier wait is bounded; on a time-out the CTA records a status code
// and unwinds through the common exit that frees its tensor memory.
#include "kernels.cuh"
#include "ptx.cuh"
#include "record.cuh"
#include "tensormap.cuh"

#include <algorithm>
#include <type_traits>
#include <cstdlib>


namespace pinkb {

namespace {

constexpr uint32_t kBlockM = 128;          // neurons per tile = TMEM lanes
constexpr uint32_t kBlockK = 128;          // bytes of K per pipeline stage = one swizzle row
constexpr uint32_t kUmmaK = 32;            // K per kind::i8 instruction
constexpr uint32_t kThreads = 192;

// PAIR: two CTAs of a cluster share one M=256 MMA (cta_group::2); each stages its own 128 neuron
// rows and only half of the transform rows, which frees shared memory for deeper rings.
template <int MODE, bool PAIR> struct TcCfg;
template <> struct TcCfg<kModeU8, false>  { static constexpr uint32_t planes = 1, max_n = 256, cols = 256; };
template <> struct TcCfg<kModeU16, false> { static constexpr uint32_t planes = 2, max_n = 128, cols = 512; };
template <> struct TcCfg<kModeU8, true>   { static constexpr uint32_t planes = 1, max_n = 256, cols = 256; };
template <> struct TcCfg<kModeU16, true>  { static constexpr uint32_t planes = 2, max_n = 128, cols = 512; };
template <> struct TcCfg<kModeTf32, false> { static constexpr uint32_t planes = 2, max_n = 256, cols = 512; };
template <> struct TcCfg<kModeTf32, true>  { static constexpr uint32_t planes = 2, max_n = 256, cols = 512; };

// Shared memory of a CTA: barriers, the tensor-memory address and the per-column |b|^2 in the first
// 4 KB, then the ring of stages.  A stage holds, per byte plane, the 128 neuron rows and this CTA's
// transform rows of one 128-byte K slice; its size follows the tile width of the launch, and the
// ring takes as many stages as fit (narrow tiles of small shards get a deeper ring, which is what
// hides the load latency when the MMAs of a slice are short).
constexpr uint32_t kMaxStages = 16;
template <int MODE, bool PAIR>
struct SmemLayout
{
    using Cfg = TcCfg<MODE, PAIR>;
    static constexpr uint32_t a_bytes = kBlockM * kBlockK;            // per plane
    static constexpr uint32_t bar_off = 0;                            // full[kMaxStages], empty[kMaxStages], tmem_full
    static constexpr uint32_t tmem_ptr_off = (2 * kMaxStages + 1) * 8;
    static constexpr uint32_t nb_off = 512;                           // per-column |b|^2 of this tile, up to 256 x 8 bytes
    static constexpr uint32_t ring_off = 4096;
    static constexpr uint32_t ring_budget = 196 * 1024;
    static constexpr uint32_t slack = 1024;                           // for the 1024-byte alignment of the base
};

struct TcParams
{
    const void* anorm;
    const void* bnorm;
    unsigned long long* keys;
    void* s_out;
    int* status;
    uint32_t n, T, num_kb, n_tile;
    uint32_t swap;              // kModeTf32 only: the transforms are the tile rows (M side), the neurons its columns
    uint32_t stages, b_bytes;   // ring depth; bytes of this CTA's transform rows per plane and stage (multiple of 1024)
    uint32_t* tail_counter;     // nullable: block arrival counter (zero between launches) that enables the tail below
    BmuArgs tail;               // the last block to finish reduces the shard's keys to its record and publishes it
};

__device__ __forceinline__ void report(int* status, int code)
{
    if (status) atomicCAS(status, kDevOk, code);
}

template <int MODE, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
distance_tc_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                   const __grid_constant__ CUtensorMap map_b0, const __grid_constant__ CUtensorMap map_b1,
                   const TcParams p)
{
    using Cfg = TcCfg<MODE, PAIR>;
    using L = SmemLayout<MODE, PAIR>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::bar_off);
    uint64_t* empty_bar = full_bar + kMaxStages;
    uint64_t* tmem_full_bar = empty_bar + kMaxStages;
    uint8_t* ring = smem + L::ring_off;
    const uint32_t stage_bytes = Cfg::planes * (L::a_bytes + p.b_bytes);
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + L::tmem_ptr_off);
    unsigned long long* nb_s = reinterpret_cast<unsigned long long*>(smem + L::nb_off);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m0 = blockIdx.x * kBlockM;
    const uint32_t t0 = blockIdx.y * p.n_tile;
    const uint32_t img = blockIdx.z;
    // PAIR: rank of this CTA in its pair (the even CTA issues the MMAs) and the transform rows it stages
    const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
    const uint32_t b_rows = PAIR ? p.n_tile / 2 : p.n_tile;
    const uint32_t stage_tx = Cfg::planes * (L::a_bytes + b_rows * kBlockK);

    if (threadIdx.x == 0) {
        // PAIR: both CTAs' producers arrive (with their byte counts) on the issuing CTA's full barriers
        for (uint32_t s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], PAIR ? 2 : 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(tmem_full_bar, 1);
        mbar_fence_init();
        tma_prefetch_desc(&map_a0);
        tma_prefetch_desc(&map_b0);
        if (Cfg::planes == 2) { tma_prefetch_desc(&map_a1); tma_prefetch_desc(&map_b1); }
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(tmem_ptr_s, Cfg::cols); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_ptr_s, Cfg::cols); tmem_relinquish(); }
    }
    tc_fence_before();
    if (PAIR) cluster_sync();             // the peer's barriers are initialised before anything arrives on them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;
    // Everything above is independent of earlier kernels; the operands, norms and keys are not.
    griddep_launch();
    griddep_wait();

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer --
        if (elect_one()) {
            // rows of the M-side map (map_a*) and of the N-side map (map_b*); swapped: the transforms of this image
            // are the M side (a tile's rows beyond T are the next image's and are never stored)
            const int32_t arow = (int32_t)(MODE == kModeTf32 && p.swap ? img * p.T + m0 : m0);
            const int32_t brow = (int32_t)(MODE == kModeTf32 && p.swap ? t0 + pair_rank * b_rows
                                                                      : img * p.T + t0 + pair_rank * b_rows);
            for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                const uint32_t s = kb % p.stages, ph = (kb / p.stages) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1)) { report(p.status, kDevTimeoutProducer); break; }
                uint8_t* st = ring + s * stage_bytes;
                const int32_t kx = (int32_t)(kb * kBlockK);
                if (PAIR) {
                    const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);      // the issuing CTA's barrier
                    mbar_expect_tx_cluster(bar, stage_tx);
                    tma_load_2d_pair(st, &map_a0, bar, kx, arow);
                    tma_load_2d_pair(st + Cfg::planes * L::a_bytes, &map_b0, bar, kx, brow);
                    if (Cfg::planes == 2) {
                        tma_load_2d_pair(st + L::a_bytes, &map_a1, bar, kx, arow);
                        tma_load_2d_pair(st + Cfg::planes * L::a_bytes + p.b_bytes, &map_b1, bar, kx, brow);
                    }
                } else {
                    mbar_expect_tx(&full_bar[s], stage_tx);
                    tma_load_2d(st, &map_a0, &full_bar[s], kx, arow);
                    tma_load_2d(st + Cfg::planes * L::a_bytes, &map_b0, &full_bar[s], kx, brow);
                    if (Cfg::planes == 2) {
                        tma_load_2d(st + L::a_bytes, &map_a1, &full_bar[s], kx, arow);
                        tma_load_2d(st + Cfg::planes * L::a_bytes + p.b_bytes, &map_b1, &full_bar[s], kx, brow);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer --
        if (pair_rank == 0 && elect_one()) {
            const uint32_t idesc = MODE == kModeTf32 ? make_idesc_tf32(PAIR ? 2 * kBlockM : kBlockM, p.n_tile)
                                                     : make_idesc_u8(PAIR ? 2 * kBlockM : kBlockM, p.n_tile);
            // PAIR: one instruction computes both CTAs' tiles; completion is signalled to both
            auto mma = [&](uint32_t d, uint64_t a, uint64_t b, uint32_t acc) {
                if (MODE == kModeTf32) { if (PAIR) umma_tf32_pair(d, a, b, idesc, acc); else umma_tf32(d, a, b, idesc, acc); }
                else if (PAIR) umma_i8_pair(d, a, b, idesc, acc);
                else umma_i8(d, a, b, idesc, acc);
            };
            auto commit = [&](uint64_t* bar) {
                if (PAIR) {
                    umma_commit_pair(smem_u32(bar));
                    umma_commit_pair(map_to_cta(smem_u32(bar), 1));
                } else {
                    umma_commit(bar);
                }
            };
            bool ok = true;
            for (uint32_t kb = 0; kb < p.num_kb && ok; ++kb) {
                const uint32_t s = kb % p.stages, ph = (kb / p.stages) & 1;
                if (!mbar_wait(&full_bar[s], ph)) { report(p.status, kDevTimeoutMma); ok = false; break; }
                tc_fence_after();
                const uint32_t st = smem_u32(ring + s * stage_bytes);
                const uint64_t a_hi = make_sw128_kmajor_desc(st);
                const uint64_t b_hi = make_sw128_kmajor_desc(st + Cfg::planes * L::a_bytes);
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k) {
                    const uint64_t adv = (k * kUmmaK) >> 4;   // 32 bytes along K inside the swizzled row
                    const uint32_t acc = (kb | k) != 0;
                    if (MODE == kModeU8) {
                        mma(tmem_base, a_hi + adv, b_hi + adv, acc);
                    } else if (MODE == kModeTf32) {
                        // the main and the cross terms share an accumulator (the cross terms are 2^-10 of the main
                        // term); even and odd K steps go to two accumulators, which halves the number of
                        // additions -- and with it the rounding -- each running sum sees
                        const uint64_t a_lo = make_sw128_kmajor_desc(st + L::a_bytes);
                        const uint64_t b_lo = make_sw128_kmajor_desc(st + Cfg::planes * L::a_bytes + p.b_bytes);
                        const uint32_t d = tmem_base + (k & 1u) * Cfg::max_n;
                        mma(d, a_hi + adv, b_hi + adv, (kb | (k >> 1)) != 0);
                        mma(d, a_hi + adv, b_lo + adv, 1u);
                        mma(d, a_lo + adv, b_hi + adv, 1u);
                    } else {
                        const uint64_t a_lo = make_sw128_kmajor_desc(st + L::a_bytes);
                        const uint64_t b_lo = make_sw128_kmajor_desc(st + Cfg::planes * L::a_bytes + p.b_bytes);
                        mma(tmem_base, a_hi + adv, b_hi + adv, acc);                         // hh
                        mma(tmem_base + Cfg::max_n, a_lo + adv, b_lo + adv, acc);            // ll
                        mma(tmem_base + 2 * Cfg::max_n, a_hi + adv, b_lo + adv, acc);        // cross
                        mma(tmem_base + 2 * Cfg::max_n, a_lo + adv, b_hi + adv, 1u);
                    }
                }
                commit(&empty_bar[s]);           // frees the stage once these MMAs have read it
            }
            commit(tmem_full_bar);               // accumulators complete
        }
    } else {
        // ----------------------------------------------------------- epilogue --
        // A thread owns one neuron row (TMEM lane) and walks the tile's columns in chunks of 16: the
        // next chunk's tcgen05.ld is in flight while the current one is reduced, and four independent
        // (minimum, column) chains keep the compare/select latency off the critical path.
        using val_t = typename std::conditional<MODE == kModeU8, uint32_t,
                      typename std::conditional<MODE == kModeTf32, float, unsigned long long>::type>::type;
        val_t* nbv = reinterpret_cast<val_t*>(nb_s);         // |b|^2 per column of this tile
        const uint32_t et = threadIdx.x - 64;               // 0..127
        const uint32_t quad = warp & 3;                      // TMEM lane quadrant this warp may read
        const uint32_t row = quad * 32 + lane;
        const uint32_t n = m0 + row;
        const bool swapped = MODE == kModeTf32 && p.swap;
        const uint32_t m_rows = swapped ? p.T : p.n, n_cols = swapped ? p.n : p.T;       // extent of the two tile sides
        const uint32_t ncols = n_cols > t0 ? min(p.n_tile, n_cols - t0) : 0u;     // columns of this tile that exist
        for (uint32_t j = et; j < p.n_tile; j += 128) {
            val_t v = 0;
            if (j < ncols) v = swapped ? static_cast<const val_t*>(p.anorm)[t0 + j]
                                       : static_cast<const val_t*>(p.bnorm)[(size_t)img * p.T + t0 + j];
            nbv[j] = v;
        }
        const val_t na = n >= m_rows ? val_t(0) : swapped ? static_cast<const val_t*>(p.bnorm)[(size_t)img * p.T + n]
                                                          : static_cast<const val_t*>(p.anorm)[n];
        asm volatile("bar.sync 1, 128;" ::: "memory");      // nbv visible to the four epilogue warps

        constexpr int kChains = 4;
        val_t best[kChains];
        uint32_t bcol[kChains];
#pragma unroll
        for (int c = 0; c < kChains; ++c) { best[c] = MODE == kModeTf32 ? val_t(0) : val_t(~0ull); bcol[c] = 0; }
        if (mbar_wait(tmem_full_bar, 0)) {
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16);
            auto load = [&](uint32_t c0, uint32_t (&x0)[16], uint32_t (&x1)[16], uint32_t (&x2)[16]) {
                tmem_ld_32x16(lane_addr + c0, x0);
                if (MODE == kModeTf32) tmem_ld_32x16(lane_addr + Cfg::max_n + c0, x1);
                if (MODE == kModeU16) {
                    tmem_ld_32x16(lane_addr + Cfg::max_n + c0, x1);
                    tmem_ld_32x16(lane_addr + 2 * Cfg::max_n + c0, x2);
                }
            };
            auto wait = [&](uint32_t (&x0)[16], uint32_t (&x1)[16], uint32_t (&x2)[16]) {
                tmem_ld_wait_on(x0);
                if (MODE == kModeTf32) tmem_ld_wait_on(x1);
                if (MODE == kModeU16) { tmem_ld_wait_on(x1); tmem_ld_wait_on(x2); }
            };
            auto reduce = [&](uint32_t c0, const uint32_t (&x0)[16], const uint32_t (&x1)[16], const uint32_t (&x2)[16]) {
                val_t sv[16];
                if (MODE == kModeTf32) {
                    // the estimate of every pair goes out (row-major per neuron: 64 contiguous bytes per thread
                    // and chunk); nothing is reduced here
                    if (swapped) {
                        // this thread's row is a transform, the columns are neurons: a warp stores 32 consecutive
                        // transforms of one neuron's row of the estimate matrix
                        if (n < p.T) {
                            float* dst = static_cast<float*>(p.s_out) + ((size_t)img * p.n + t0 + c0) * p.T + n;
#pragma unroll
                            for (uint32_t j = 0; j < 16; ++j)
                                if (c0 + j < ncols)
                                    dst[(size_t)j * p.T] = fmaxf((float)na + (float)nbv[c0 + j]
                                                                 - 2.0f * (__uint_as_float(x0[j]) + __uint_as_float(x1[j])), 0.0f);
                        }
                    } else if (n < p.n) {
                        float* dst = static_cast<float*>(p.s_out) + ((size_t)img * p.n + n) * p.T + t0 + c0;
#pragma unroll
                        for (uint32_t j = 0; j < 16; j += 4) {
                            float4 o;
                            o.x = fmaxf((float)na + (float)nbv[c0 + j] - 2.0f * (__uint_as_float(x0[j]) + __uint_as_float(x1[j])), 0.0f);
                            o.y = fmaxf((float)na + (float)nbv[c0 + j + 1] - 2.0f * (__uint_as_float(x0[j + 1]) + __uint_as_float(x1[j + 1])), 0.0f);
                            o.z = fmaxf((float)na + (float)nbv[c0 + j + 2] - 2.0f * (__uint_as_float(x0[j + 2]) + __uint_as_float(x1[j + 2])), 0.0f);
                            o.w = fmaxf((float)na + (float)nbv[c0 + j + 3] - 2.0f * (__uint_as_float(x0[j + 3]) + __uint_as_float(x1[j + 3])), 0.0f);
                            // rows of T floats: 16-byte stores only where every row starts on a 16-byte boundary
                            if ((p.T & 3u) == 0 && c0 + j + 4 <= ncols) *reinterpret_cast<float4*>(dst + j) = o;
                            else {
                                if (c0 + j < ncols) dst[j] = o.x;
                                if (c0 + j + 1 < ncols) dst[j + 1] = o.y;
                                if (c0 + j + 2 < ncols) dst[j + 2] = o.z;
                                if (c0 + j + 3 < ncols) dst[j + 3] = o.w;
                            }
                        }
                    }
                } else {
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) {
                    if (MODE == kModeU8) {
                        // exact: 0 <= S < 2^31 although the intermediates wrap modulo 2^32
                        sv[j] = (uint32_t)(na + nbv[c0 + j]) - 2u * x0[j];
                    } else if (MODE == kModeU16) {
                        const unsigned long long dot = ((unsigned long long)x0[j] << 16)
                                                     + ((unsigned long long)x2[j] << 8) + x1[j];
                        sv[j] = na + nbv[c0 + j] - 2ull * dot;
                    } else {
                        sv[j] = 0;
                    }
                }
                if (c0 + 16 > ncols) {                        // ragged last chunk: columns beyond T never win
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j) if (c0 + j >= ncols) sv[j] = val_t(~0ull);
                }
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j)
                    if (sv[j] < best[j % kChains]) { best[j % kChains] = sv[j]; bcol[j % kChains] = c0 + j; }
                if (p.s_out && n < p.n) {
#pragma unroll
                    for (uint32_t j = 0; j < 16; ++j)
                        if (c0 + j < ncols)
                            static_cast<val_t*>(p.s_out)[((size_t)img * p.n + n) * p.T + t0 + c0 + j] = sv[j];
                }
                }
            };
            uint32_t a0[16], a1[16], a2[16], b0[16], b1[16], b2[16];
            if (ncols) load(0, a0, a1, a2);
            for (uint32_t c0 = 0; c0 < ncols; c0 += 32) {
                wait(a0, a1, a2);
                if (c0 + 16 < ncols) load(c0 + 16, b0, b1, b2);
                reduce(c0, a0, a1, a2);
                if (c0 + 16 < ncols) {
                    wait(b0, b1, b2);
                    if (c0 + 32 < ncols) load(c0 + 32, a0, a1, a2);
                    reduce(c0 + 16, b0, b1, b2);
                }
            }
            // first minimum over the chains: lowest S, then lowest column
            val_t best_s = best[0];
            uint32_t best_c = bcol[0];
#pragma unroll
            for (int c = 1; c < kChains; ++c)
                if (best[c] < best_s || (best[c] == best_s && bcol[c] < best_c)) { best_s = best[c]; best_c = bcol[c]; }
            if (MODE != kModeTf32 && n < p.n && best_s != val_t(~0ull))
                atomicMin(&p.keys[(size_t)img * p.n + n],
                          ((unsigned long long)best_s << key_shift(MODE)) | (unsigned long long)(t0 + best_c));
        } else {
            report(p.status, kDevTimeoutEpilogue);
        }
    }

    tc_fence_before();
    if (PAIR) cluster_sync();             // neither CTA leaves while the other may still signal or read it
    else __syncthreads();
    if (warp == 1) {
        if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::cols); else tmem_dealloc(tmem_base, Cfg::cols);
    }

    // Tail (training with several ranks): the block that finishes last has all per-neuron minima in
    // front of it; it reduces them to this shard's best-matching-unit record and hands the record to the
    // other ranks, which saves a kernel of its own between this one and the update.
    if (p.tail_counter) {
        __shared__ uint32_t last_s;
        __shared__ unsigned long long tc_s[kThreads / 32], tn_s[kThreads / 32];
        if (threadIdx.x == 0) {
            __threadfence();                                   // this block's key updates before its arrival
            const uint32_t blocks = gridDim.x * gridDim.y * gridDim.z;
            const uint32_t old = atomicAdd(p.tail_counter, 1u);
            last_s = old == blocks - 1;
            if (old == blocks - 1) *p.tail_counter = 0;
            __threadfence();
        }
        __syncthreads();
        if (last_s) {
            unsigned long long bc, bn;
            block_argmin_keys(p.tail.keys, p.tail.n, p.tail.shift, kThreads, tc_s, tn_s, bc, bn);
            __syncthreads();
            if (threadIdx.x == 0) { tc_s[0] = bc; tn_s[0] = bn == ~0ull ? ~0ull : shard_global(p.tail.first_neuron, p.tail.neuron_stride, bn); }
            __syncthreads();
            publish_record(p.tail, tc_s[0], tn_s[0]);
        }
    }
}

// ------------------------------------------------------------------ host side --

template <int MODE, bool PAIR>
cudaError_t launch_tc(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why, bool swap = false)
{
    using Cfg = TcCfg<MODE, PAIR>;
    using L = SmemLayout<MODE, PAIR>;
    // The tile rows (M side, 128 per block) are the neurons and the tile columns the transforms -- or, swapped
    // (float estimate only), the other way round.
    const uint32_t m_extent = swap ? g.T : a.n, n_extent = swap ? a.n : g.T;
    // row tiles; CTA pairs take two consecutive ones (an odd count is padded with an empty tile)
    uint32_t m_tiles = (m_extent + kBlockM - 1) / kBlockM;
    if (PAIR) m_tiles = (m_tiles + 1) & ~1u;
    // Balanced column tiles, each a multiple of 16 columns: the fewest tiles of at most max_n
    // columns -- unless that leaves SMs without a block (a small neuron shard, few images): a block's
    // run time is set by the bytes it pulls through its SM, (128 + its share of n_tile) * K, so narrower
    // tiles spread over all SMs finish sooner.  Below 32 columns the row tile dominates and nothing is gained.
    uint32_t tiles = (n_extent + Cfg::max_n - 1) / Cfg::max_n;
    {
        static thread_local int sm_dev = -1, sms = 0;
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev != sm_dev) { cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); sm_dev = dev; }
        const uint64_t rows = (uint64_t)m_tiles * a.n_img;
        const uint32_t most = std::max<uint32_t>(tiles, n_extent / 32);
        if (sms > 0 && rows * tiles < (uint64_t)sms)
            tiles = (uint32_t)std::max<uint64_t>(tiles, std::min<uint64_t>(most, (uint64_t)sms / rows));   // one wave
    }
    uint32_t n_tile = ((n_extent + tiles - 1) / tiles + 15) & ~15u;
    if (n_tile > Cfg::max_n) n_tile = Cfg::max_n;
    const uint32_t n_tiles = (n_extent + n_tile - 1) / n_tile;
    const uint32_t b_box = PAIR ? n_tile / 2 : n_tile;         // column-side rows one CTA stages per K slice

    CUtensorMap ma0, ma1, mb0, mb1;
    const uint64_t row_bytes = MODE == kModeTf32 ? 4ull * g.Kp : g.Kp;      // Kp counts operand elements
    const uint64_t som_rows = a.n, tr_rows = (uint64_t)a.n_img * g.T;
    bool ok = swap ? make_map(&ma0, a.b0, tr_rows, row_bytes, kBlockM) && make_map(&mb0, a.a0, som_rows, row_bytes, b_box)
                   : make_map(&ma0, a.a0, som_rows, row_bytes, kBlockM) && make_map(&mb0, a.b0, tr_rows, row_bytes, b_box);
    if (Cfg::planes == 2)
        ok = ok && (swap ? make_map(&ma1, a.b1, tr_rows, row_bytes, kBlockM) && make_map(&mb1, a.a1, som_rows, row_bytes, b_box)
                         : make_map(&ma1, a.a1, som_rows, row_bytes, kBlockM) && make_map(&mb1, a.b1, tr_rows, row_bytes, b_box));
    else { ma1 = ma0; mb1 = mb0; }
    if (!ok) { *why = "cuTensorMapEncodeTiled failed"; return cudaErrorInvalidValue; }

    static thread_local int attr_dev = -1;   // the opt-in shared-memory size is a per-device function attribute
    int dev = 0;
    cudaGetDevice(&dev);
    constexpr uint32_t smem_max = L::ring_off + L::ring_budget + L::slack;
    if (dev != attr_dev) {
        cudaError_t e = cudaFuncSetAttribute(distance_tc_kernel<MODE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem_max);
        if (e != cudaSuccess) { *why = "cudaFuncSetAttribute(distance_tc_kernel)"; return e; }
        attr_dev = dev;
    }
    // ring: as many stages as fit the budget, no more than there are K slices
    const uint32_t b_bytes = (b_box * kBlockK + 1023) & ~1023u;
    const uint32_t stage_bytes = Cfg::planes * (L::a_bytes + b_bytes);
    const uint32_t num_kb = (uint32_t)(row_bytes / kBlockK);
    uint32_t stages = std::max(2u, std::min(std::min(kMaxStages, L::ring_budget / stage_bytes), num_kb));
    {
        // More blocks than SMs (mapping: a batch of images per launch): a ring of three stages is as good as a deeper
        // one when a second block of the same kernel shares the SM -- one block's epilogue and first loads then hide
        // behind the other's main loop (measured: 57 k instead of 49 k images/s mapping uint8 at 2791 x 1440 x 4096).
        // Only where both blocks' accumulators fit the tensor memory (256 columns each).
        static thread_local int sm_dev2 = -1, sms2 = 0;
        int dev2 = 0;
        cudaGetDevice(&dev2);
        if (dev2 != sm_dev2) { cudaDeviceGetAttribute(&sms2, cudaDevAttrMultiProcessorCount, dev2); sm_dev2 = dev2; }
        constexpr uint32_t half_sm = 113u * 1024u;                       // shared memory of one of two resident blocks
        const uint64_t blocks = (uint64_t)m_tiles * n_tiles * a.n_img;
        if (Cfg::cols <= 256 && sms2 > 0 && blocks > (uint64_t)sms2 && stages > 3
            && L::ring_off + 3 * stage_bytes + L::slack <= half_sm)
            stages = std::min(stages, (half_sm - L::ring_off - L::slack) / stage_bytes);
    }
    TcParams p;
    p.anorm = a.anorm; p.bnorm = a.bnorm; p.keys = a.keys; p.s_out = a.s_out; p.status = a.status;
    p.n = a.n; p.T = g.T; p.num_kb = num_kb; p.n_tile = n_tile; p.swap = swap ? 1u : 0u;
    p.stages = stages; p.b_bytes = b_bytes;
    p.tail_counter = a.tail ? a.tail_counter : nullptr;
    if (a.tail) p.tail = *a.tail;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m_tiles, n_tiles, a.n_img);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::ring_off + stages * stage_bytes + L::slack;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // the kernel's set-up may overlap the tail of the kernel before it in the stream (it waits
    // with griddepcontrol.wait before it touches global memory)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    *why = "distance_tc_kernel launch";
    return cudaLaunchKernelEx(&cfg, distance_tc_kernel<MODE, PAIR>, ma0, ma1, mb0, mb1, p);
}

// CTA pairs halve the transform rows every SM pulls through its L2 port (the kernel's bound) as soon
// as there are two neuron tiles to pair.  DistanceArgs::single_cta (diagnostic switch) keeps single CTAs.
template <int MODE>
cudaError_t launch_tc_any(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why)
{
    if (a.n > kBlockM && !a.single_cta) return launch_tc<MODE, true>(g, a, st, why);
    return launch_tc<MODE, false>(g, a, st, why);
}

} // namespace

cudaError_t launch_distance_f32(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why);

// float32 filter pass: a0/a1 and b0/b1 are the TF32 word planes (high, low) of the operands, anorm/bnorm float
// |.|^2, s_out [n_img][n][T] float receives the estimates; keys are not touched.  Needs Kp % 32 == 0.
cudaError_t launch_distance_tf32(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why)
{
    *why = "";
    if (a.n == 0 || a.n_img == 0) return cudaSuccess;
    if (g.Kp % 32 != 0 || !a.s_out) { *why = "launch_distance_tf32: operand stride or output"; return cudaErrorInvalidValue; }
    // orientation: the one whose padded tile grid (rows to 128, or 256 for block pairs; columns to balanced tiles of
    // at most 256, multiples of 16) computes fewer pairs that do not exist
    auto padded = [](uint32_t m, uint32_t n) -> uint64_t {
        const uint32_t mp = m > kBlockM ? (m + 2 * kBlockM - 1) / (2 * kBlockM) * (2 * kBlockM) : kBlockM;
        const uint32_t tiles = (n + 255) / 256, nt = (((n + tiles - 1) / tiles) + 15) & ~15u;
        return (uint64_t)mp * ((n + nt - 1) / nt) * nt;
    };
    const bool swap = padded(g.T, a.n) < padded(a.n, g.T);
    const uint32_t m_extent = swap ? g.T : a.n;
    if (m_extent > kBlockM && !a.single_cta) return launch_tc<kModeTf32, true>(g, a, st, why, swap);
    return launch_tc<kModeTf32, false>(g, a, st, why, swap);
}

bool distance_has_tail(const Geometry& g) { return g.mode == kModeU8 || g.mode == kModeU16; }

cudaError_t launch_distance(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why)
{
    *why = "";
    if (a.n == 0 || a.n_img == 0) return cudaSuccess;
    if (g.mode == kModeU8) return launch_tc_any<kModeU8>(g, a, st, why);
    if (g.mode == kModeU16) return launch_tc_any<kModeU16>(g, a, st, why);
    return launch_distance_f32(g, a, st, why);
}

} // namespace pinkb
