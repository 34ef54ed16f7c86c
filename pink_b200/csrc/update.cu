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

__global__ void __launch_bounds__(1024)
bmu_kernel(const unsigned long long* __restrict__ keys, uint32_t n, uint32_t first_neuron, uint32_t shift,
           BmuPair* __restrict__ out)
{
    __shared__ unsigned long long sc[32], sn[32];
    unsigned long long bc = ~0ull, bn = ~0ull;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        unsigned long long c = keys[i] >> shift;
        if (pair_less(c, i, bc, bn)) { bc = c; bn = i; }
    }
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
        if (lane == 0) { out->code = bc; out->neuron = bn == ~0ull ? ~0ull : bn + first_neuron; }
    }
}

template <int MODE>
__global__ void __launch_bounds__(256)
update_kernel(Geometry g, UpdateArgs a, uint32_t stage_base)
{
    extern __shared__ __align__(16) uint8_t dyn[];
    float* base_s = reinterpret_cast<float*>(dyn);                       // [P] base rotation (all channels)
    uint8_t* crop_s = dyn + (stage_base ? (((size_t)g.P * 4 + 15) & ~size_t(15)) : 0);   // operand row(s) being rebuilt
    __shared__ unsigned long long red[8];
    __shared__ unsigned long long key_s;
    __shared__ uint32_t bmu_s;

    const uint32_t n = blockIdx.x;
    if (threadIdx.x == 0) {
        // Global best matching unit: lexicographic minimum over the per-rank records.
        unsigned long long bc = a.pairs[0].code, bn = a.pairs[0].neuron;
        for (uint32_t r = 1; r < a.world; ++r)
            if (pair_less(a.pairs[r].code, a.pairs[r].neuron, bc, bn)) { bc = a.pairs[r].code; bn = a.pairs[r].neuron; }
        bmu_s = (uint32_t)bn;
        key_s = a.keys[n];
        a.keys[n] = kKeyEmpty;      // re-arm for the next image's distance kernel
    }
    __syncthreads();
    const uint32_t bmu = bmu_s;
    if (threadIdx.x == 0 && a.first_neuron + n == bmu) {
        atomicAdd(&a.counts[bmu], 1u);
        if (a.bmu_log) *a.bmu_log = bmu;
    }
    const float f = a.factors[(size_t)bmu * a.n + n];
    if (f == 0.0f) return;           // uniform for the block

    // Decode the best transform into (flip, quadrant, base rotation).
    const uint32_t t = (uint32_t)(key_s & ((1ull << key_shift(MODE)) - 1));
    const uint32_t fl = t / g.R, r = t - fl * g.R;
    const uint32_t j = g.q ? r / g.q : 0, tq = g.q ? r - j * g.q : 0;
    const float* base = a.base + (size_t)tq * g.P;

    // Stage the base rotation in shared memory when it fits; otherwise read it
    // through the read-only cache (it is shared by all neurons and L2 resident).
    const float* bsrc = base;
    if (stage_base) {
        if ((g.P & 3) == 0) {
            for (uint32_t i = threadIdx.x; i < g.P / 4; i += blockDim.x)
                reinterpret_cast<float4*>(base_s)[i] = __ldg(reinterpret_cast<const float4*>(base) + i);
        } else {
            for (uint32_t i = threadIdx.x; i < g.P; i += blockDim.x) base_s[i] = __ldg(base + i);
        }
        __syncthreads();
        bsrc = base_s;
    }

    float* w = a.som + (size_t)n * g.Pp;
    const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    const uint32_t nd1 = g.nd - 1;
    unsigned long long acc = 0;
    for (uint32_t i4 = threadIdx.x; i4 < g.Pp / 4; i4 += blockDim.x) {
        float4 v = reinterpret_cast<float4*>(w)[i4];
        float e[4] = { v.x, v.y, v.z, v.w };
        uint32_t idx = i4 * 4;
        uint32_t c = idx / P1, rem = idx - c * P1;
        uint32_t x = rem / g.nd, y = rem - x * g.nd;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (idx + k < g.P) {
                uint32_t sx = fl ? nd1 - x : x, bx, by;
                switch (j) {
                    case 0: bx = sx; by = y; break;
                    case 1: bx = nd1 - y; by = sx; break;
                    case 2: bx = nd1 - sx; by = nd1 - y; break;
                    default: bx = y; by = nd1 - sx; break;
                }
                const float rv = bsrc[c * P1 + bx * g.nd + by];
                const float nv = __fsub_rn(e[k], __fmul_rn(__fsub_rn(e[k], rv), f));
                e[k] = nv;
                const uint32_t ci = x - g.off, cj = y - g.off;    // unsigned wrap rejects x < off
                if (ci < g.ed && cj < g.ed) {
                    const uint32_t kk = c * K1 + ci * g.ed + cj;
                    if (MODE == kModeU8) {
                        uint32_t qv = quant_u8(nv);
                        crop_s[kk] = (uint8_t)qv;
                        acc += qv * qv;
                    } else if (MODE == kModeU16) {
                        uint32_t qv = quant_u16(nv);
                        crop_s[kk] = (uint8_t)(qv >> 8);
                        crop_s[g.Kp + kk] = (uint8_t)(qv & 255);
                        acc += (unsigned long long)qv * qv;
                    } else {
                        reinterpret_cast<float*>(crop_s)[kk] = nv;
                    }
                }
            }
            if (++y == g.nd) { y = 0; if (++x == g.nd) { x = 0; ++c; } }
        }
        reinterpret_cast<float4*>(w)[i4] = make_float4(e[0], e[1], e[2], e[3]);
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
    const size_t crop = MODE == kModeF32 ? (size_t)g.Kp * 4 : (MODE == kModeU16 ? (size_t)g.Kp * 2 : g.Kp);
    const size_t staged = (((size_t)g.P * 4 + 15) & ~size_t(15)) + crop;
    const uint32_t stage_base = staged <= 200 * 1024;
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
    update_kernel<MODE><<<a.n, 256, smem, st>>>(g, a, stage_base);
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_bmu(const Geometry& g, const unsigned long long* keys, uint32_t n, uint32_t first_neuron,
                       BmuPair* out, cudaStream_t st)
{
    bmu_kernel<<<1, 1024, 0, st>>>(keys, n, first_neuron, key_shift(g.mode), out);
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
