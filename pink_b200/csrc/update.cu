// Best-matching-unit reduction, neighbourhood update and mapping epilogue.
//
// bmu_kernel replaces find_best_matching_neuron_kernel, a single-thread serial
// scan followed by a device-to-host read (src/CudaLib/update_neurons.h:18-31,
// :64-80), by one block-wide first-minimum reduction whose result stays on the
// device.
//
// update_kernel replaces update_neurons_kernel (src/CudaLib/update_neurons.h:
// 34-49) and, in the same pass, the next image's copy_and_transform_kernel over
// the SOM (src/CudaLib/generate_euclidean_distance_matrix.h:64-84): one CTA per
// neuron loads the base rotation its best transform derives from into shared
// memory, applies  w <- w - (w - r) * f  with 128-bit loads and stores, reading
// r through the quarter-turn/flip index permutation instead of from a
// materialised T x P array, and re-emits the neuron's quantised distance
// operand row and its sum of squares.  The difference, the product and the
// final subtraction are rounded separately (never contracted to FMA), as in
// the reference's CPU loop (src/SelfOrganizingMapLib/Trainer.h:167-179).
#include "kernels.cuh"
#include "ptx.cuh"

namespace pinkb {

namespace {

__device__ __forceinline__ uint32_t quant_u8(float v)
{
    return min(__float2uint_rz(__fmul_rn(v, 255.0f)), 255u);
}

__device__ __forceinline__ uint32_t quant_u16(float v)
{
    return min(__float2uint_rz(__fmul_rn(v, 65535.0f)), 65535u);
}

__device__ __forceinline__ bool pair_less(unsigned long long c0, unsigned long long n0,
                                          unsigned long long c1, unsigned long long n1)
{
    return c0 < c1 || (c0 == c1 && n0 < n1);
}

// Block-wide first minimum of (code, index) pairs held one per thread.
__device__ __forceinline__ void block_min_pair(unsigned long long& bc, unsigned long long& bn,
                                               unsigned long long* sc, unsigned long long* sn)
{
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
        if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sc[warp] = bc; sn[warp] = bn; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        bc = lane < nw ? sc[lane] : ~0ull;
        bn = lane < nw ? sn[lane] : ~0ull;
        for (int o = 16; o > 0; o >>= 1) {
            unsigned long long oc = __shfl_down_sync(0xffffffffu, bc, o), on = __shfl_down_sync(0xffffffffu, bn, o);
            if (pair_less(oc, on, bc, bn)) { bc = oc; bn = on; }
        }
    }
}

// One block.  phase bit 0: reduce this shard's keys to its (code, neuron)
// record; phase bit 1: pick the global best matching unit from the per-rank
// records, count the hit, and compact the shard's neurons whose update factor
// for that unit is non-zero into (active, f_active, n_active), in ascending
// neuron order.  A single-GPU step runs both phases in one launch; with
// several ranks the exchange of the records sits between them.
__global__ void __launch_bounds__(1024)
bmu_kernel(BmuArgs a, uint32_t phase)
{
    __shared__ unsigned long long sc[32], sn[32];
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t bmu_s, base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (phase & 1u) {
        unsigned long long bc = ~0ull, bn = ~0ull;
        for (uint32_t i = threadIdx.x; i < a.n; i += blockDim.x) {
            unsigned long long c = a.keys[i] >> a.shift;
            if (pair_less(c, i, bc, bn)) { bc = c; bn = i; }
        }
        block_min_pair(bc, bn, sc, sn);
        if (threadIdx.x == 0) {
            a.pairs[a.rank].code = bc;
            a.pairs[a.rank].neuron = bn == ~0ull ? ~0ull : bn + a.first_neuron;
        }
        if (!(phase & 2u)) return;
        __syncthreads();
    }

    if (threadIdx.x == 0) {
        unsigned long long bc = a.pairs[0].code, bn = a.pairs[0].neuron;
        for (uint32_t r = 1; r < a.world; ++r)
            if (pair_less(a.pairs[r].code, a.pairs[r].neuron, bc, bn)) { bc = a.pairs[r].code; bn = a.pairs[r].neuron; }
        const uint32_t bmu = (uint32_t)bn;
        bmu_s = bmu;
        base_s = 0;
        if (bmu >= a.first_neuron && bmu - a.first_neuron < a.n) {      // this rank owns the unit
            a.counts[bmu] += 1;
            if (a.bmu_log) *a.bmu_log = bmu;
        }
    }
    __syncthreads();
    const float* frow = a.factors + (size_t)bmu_s * a.n;
    for (uint32_t i0 = 0; i0 < a.n; i0 += blockDim.x) {
        const uint32_t i = i0 + threadIdx.x;
        const float f = i < a.n ? frow[i] : 0.0f;
        const bool on = f != 0.0f;
        const uint32_t ballot = __ballot_sync(0xffffffffu, on);
        if (lane == 0) warp_tot[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = base_s;
        for (int w = 0; w < warp; ++w) before += warp_tot[w];
        if (i < a.n) {
            const unsigned long long key = a.keys[i];
            a.keys[i] = kKeyEmpty;        // re-arm every key for the next image's distance kernel
            if (on) {
                const uint32_t slot = before + __popc(ballot & ((1u << lane) - 1));
                a.active[slot] = i;
                a.f_active[slot] = f;
                a.t_active[slot] = (uint32_t)(key & ((1ull << a.shift) - 1));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t tot = 0;
            for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) tot += warp_tot[w];
            base_s += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *a.n_active = base_s;
}

constexpr int kUpdVec = 8;            // float4 loads a thread keeps in flight
constexpr int kUpdThreads = 256;

// Flat element index -> (row over all channels, column) with a multiply-high;
// exact while idx * nd < 2^32 (checked on the host).
__device__ __forceinline__ uint32_t fast_div(uint32_t v, uint32_t magic) { return __umulhi(v, magic); }

template <int MODE>
__global__ void __launch_bounds__(kUpdThreads, 3)
update_kernel(Geometry g, UpdateArgs a, uint32_t stage_base, uint32_t magic_nd)
{
    extern __shared__ __align__(16) uint8_t dyn[];
    float* base_s = reinterpret_cast<float*>(dyn);                       // [P] base rotation (all channels)
    uint8_t* crop_s = dyn + (stage_base ? (((size_t)g.P * 4 + 15) & ~size_t(15)) : 0);   // operand row(s) being rebuilt
    __shared__ __align__(8) uint64_t bar;
    __shared__ unsigned long long red[8];
    __shared__ uint32_t n_s, t_s, coef_s[4];
    __shared__ float f_s;

    if (threadIdx.x == 0) {
        // independent loads; entries beyond n_active are stale but in bounds
        const uint32_t cnt = *a.n_active, n = a.active[blockIdx.x], t = a.t_active[blockIdx.x];
        f_s = a.f_active[blockIdx.x];
        t_s = t;
        n_s = blockIdx.x < cnt ? n : ~0u;
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t n = n_s;
    if (n == ~0u) return;                 // fewer active neurons than blocks
    const float f = f_s;

    // Everything this block will read from the SOM goes in flight before any
    // dependent work: kUpdVec 128-bit loads per thread.
    float* w = a.som + (size_t)n * g.Pp;
    const uint32_t nvec = g.Pp / 4;
    float4 v[kUpdVec];
#pragma unroll
    for (int u = 0; u < kUpdVec; ++u) {
        const uint32_t i4 = threadIdx.x + u * kUpdThreads;
        if (i4 < nvec) v[u] = __ldcs(reinterpret_cast<const float4*>(w) + i4);
    }

    // Best transform -> (flip, quadrant, base rotation) and the affine map
    // src = c*nd*nd + ax*x + ay*y + a0 from a neuron pixel (x, y) to the base
    // rotation: flip reverses rows last (src/CudaLib/flip_kernel.h:28), a
    // quarter turn maps (x, y) <- (nd-1-y, x) (src/CudaLib/rotate_90_degrees_list.h:28).
    if (threadIdx.x == 0) {
        const uint32_t t = t_s;
        const uint32_t fl = t / g.R, r = t - fl * g.R;
        const uint32_t j = g.q ? r / g.q : 0, tq = g.q ? r - j * g.q : 0;
        const int32_t nd = (int32_t)g.nd, nd1 = nd - 1;
        int32_t ax, ay, a0;
        switch (j) {
            case 0:  ax = fl ? -nd : nd; ay = 1;   a0 = fl ? nd1 * nd : 0; break;
            case 1:  ax = fl ? -1 : 1;   ay = -nd; a0 = nd1 * nd + (fl ? nd1 : 0); break;
            case 2:  ax = fl ? nd : -nd; ay = -1;  a0 = fl ? nd1 : nd1 * nd + nd1; break;
            default: ax = fl ? 1 : -1;   ay = nd;  a0 = fl ? 0 : nd1; break;
        }
        coef_s[0] = (uint32_t)ax; coef_s[1] = (uint32_t)ay; coef_s[2] = (uint32_t)a0; coef_s[3] = tq;
        if (stage_base) {
            // one bulk asynchronous copy (TMA) of the whole base rotation into shared memory
            mbar_expect_tx(&bar, g.P * 4);
            bulk_load(base_s, a.base + (size_t)tq * g.P, g.P * 4, &bar);
        }
    }
    __syncthreads();
    const int32_t ax = (int32_t)coef_s[0], ay = (int32_t)coef_s[1], a0 = (int32_t)coef_s[2];
    const float* bsrc = a.base + (size_t)coef_s[3] * g.P;
    if (stage_base) {
        if (!mbar_wait(&bar, 0)) return;  // bounded; cannot expire unless the copy faulted
        bsrc = base_s;
    }

    const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    unsigned long long acc = 0;
    for (uint32_t chunk = 0; chunk < nvec; chunk += kUpdVec * kUpdThreads) {
        if (chunk) {
#pragma unroll
            for (int u = 0; u < kUpdVec; ++u) {
                const uint32_t i4 = chunk + threadIdx.x + u * kUpdThreads;
                if (i4 < nvec) v[u] = __ldcs(reinterpret_cast<const float4*>(w) + i4);
            }
        }
#pragma unroll
        for (int u = 0; u < kUpdVec; ++u) {
            const uint32_t i4 = chunk + threadIdx.x + u * kUpdThreads;
            if (i4 >= nvec) break;
            float e[4] = { v[u].x, v[u].y, v[u].z, v[u].w };
            const uint32_t idx = i4 * 4;
            uint32_t row = fast_div(idx, magic_nd);            // c * nd + x
            uint32_t y = idx - row * g.nd;
            uint32_t c = fast_div(row, magic_nd), x = row - c * g.nd;
            int32_t s = (int32_t)(c * P1) + ax * (int32_t)x + ay * (int32_t)y + a0;
            uint32_t ci = x - g.off;                             // unsigned wrap rejects x < off
            uint32_t kk = c * K1 + ci * g.ed - g.off;            // + y gives the operand position
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (idx + k < g.P) {
                    const float rv = bsrc[s];
                    const float nv = __fsub_rn(e[k], __fmul_rn(__fsub_rn(e[k], rv), f));
                    e[k] = nv;
                    if (ci < g.ed && y - g.off < g.ed) {
                        if (MODE == kModeU8) {
                            const uint32_t qv = quant_u8(nv);
                            crop_s[kk + y] = (uint8_t)qv;
                            acc += qv * qv;
                        } else if (MODE == kModeU16) {
                            const uint32_t qv = quant_u16(nv);
                            crop_s[kk + y] = (uint8_t)(qv >> 8);
                            crop_s[g.Kp + kk + y] = (uint8_t)(qv & 255);
                            acc += (unsigned long long)qv * qv;
                        } else {
                            reinterpret_cast<float*>(crop_s)[kk + y] = nv;
                        }
                    }
                }
                ++y; s += ay;
                if (y == g.nd) {                                 // next row (and possibly next channel)
                    y = 0; ++x;
                    if (x == g.nd) { x = 0; ++c; }
                    s = (int32_t)(c * P1) + ax * (int32_t)x + a0;
                    ci = x - g.off;
                    kk = c * K1 + ci * g.ed - g.off;
                }
            }
            __stcs(reinterpret_cast<float4*>(w) + i4, make_float4(e[0], e[1], e[2], e[3]));
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
cudaError_t update_dispatch(const Geometry& g, const UpdateArgs& a, cudaStream_t st)
{
    if ((uint64_t)g.P * g.nd >= (1ull << 32)) return cudaErrorInvalidValue;   // multiply-high division range
    const size_t crop = MODE == kModeF32 ? (size_t)g.Kp * 4 : (MODE == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    const size_t staged = (((size_t)g.P * 4 + 15) & ~size_t(15)) + crop;
    // The bulk copy needs a size that is a multiple of 16 bytes; otherwise (and
    // when a base rotation does not fit) the base is read through the cache.
    const uint32_t stage_base = staged <= 200 * 1024 && (g.P & 3) == 0;
    const size_t smem = stage_base ? staged : crop;
    // Dynamic shared memory above 48 KB is an opt-in, per-device function attribute.
    static int attr_dev = -1;
    static size_t attr_bytes = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev != attr_dev || smem > attr_bytes)) {
        cudaError_t e = cudaFuncSetAttribute(update_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
        attr_bytes = smem;
    }
    const uint32_t magic = (uint32_t)((1ull << 32) / g.nd) + 1;
    update_kernel<MODE><<<a.n, kUpdThreads, smem, st>>>(g, a, stage_base, magic);
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_bmu(const BmuArgs& a, uint32_t phase, cudaStream_t st)
{
    bmu_kernel<<<1, 512, 0, st>>>(a, phase);
    return cudaGetLastError();
}

cudaError_t launch_update(const Geometry& g, const UpdateArgs& a, cudaStream_t st)
{
    if (a.n == 0) return cudaSuccess;
    if (g.mode == kModeU8) return update_dispatch<kModeU8>(g, a, st);
    if (g.mode == kModeU16) return update_dispatch<kModeU16>(g, a, st);
    return update_dispatch<kModeF32>(g, a, st);
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
