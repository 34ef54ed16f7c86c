// float32 mapping as a tensor-core filter followed by an exact pass.
//
// The reference computes every one of the N x T float distances with direct differences
// (src/CudaLib/euclidean_distance_kernel.h:61-102, CPU: src/ImageProcessingLib/euclidean_distance.h:60-64) and then
// keeps the minimum per neuron (generate_euclidean_distance_matrix_second_step.h:18-38).  Only that minimum and
// its transform leave the Mapper (src/SelfOrganizingMapLib/Mapper.h:181-208), so here the full matrix is
// computed only approximately -- as |a|^2 + |b|^2 - 2 a.b with the dot products on the tensor cores
// (distance_tc.cu, kind::tf32 on operands split into two TF32 words) -- and the exact direct-difference sum is
// evaluated for the transforms the estimate cannot rule out.  The reported distance is always an exact sum, so
// its accuracy is that of the float kernel; the estimate only decides which sums are formed.
//
// Error bound of the estimate, relative to |a|^2 + |b|^2 (which bounds 2 * sum |a_k b_k|):
//   operands: a = ah + al with ah the top 19 bits and al = a - ah (exact); the tensor core reads the top 19 bits of
//   al again, so each operand is off by at most 2^-20 of itself, and the dropped al.bl term is below 2^-20 |a_k b_k|:
//   together below 2^-18;
//   inside an instruction (eight products of one K step): at most eight roundings of a partial sum that is itself
//   one K step's share of the total: below 2^-20 summed over the steps;
//   accumulation: each of the 3 * K / 8 instructions adds its result into a float accumulator once, and that
//   addition may lose one unit in the last place of the running sum even if the unit truncates (observed: it
//   does).  Even and odd K steps use separate accumulators, so an accumulator sees 3 * K / 16 additions of its own
//   part of the sum: 3 * K / 16 * 2^-23 of the whole.
// eps = 3 * K / 16 * 2^-23 + 2^-17.  The largest deviation seen among the evaluated pairs is recorded so that tests
// can compare it with eps (C2: 0.3 of eps).
#include "kernels.cuh"

namespace pinkb {

namespace {

constexpr uint32_t kSplitThreads = 256;

__global__ void __launch_bounds__(kSplitThreads)
split_tf32_kernel(const float* __restrict__ src, uint32_t Kp, float* __restrict__ hi, float* __restrict__ lo,
                  float* __restrict__ norm)
{
    const size_t row = blockIdx.x;
    const float4* s4 = reinterpret_cast<const float4*>(src + row * Kp);
    float4* h4 = reinterpret_cast<float4*>(hi + row * Kp);
    float4* l4 = reinterpret_cast<float4*>(lo + row * Kp);
    double acc = 0.0;
    for (uint32_t i = threadIdx.x; i < Kp / 4; i += kSplitThreads) {
        const float4 v = s4[i];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u); l.x = __fsub_rn(v.x, h.x);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u); l.y = __fsub_rn(v.y, h.y);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u); l.z = __fsub_rn(v.z, h.z);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u); l.w = __fsub_rn(v.w, h.w);
        h4[i] = h;
        l4[i] = l;
        acc += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
    __shared__ double part[kSplitThreads / 32];
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (uint32_t w = 0; w < kSplitThreads / 32; ++w) tot += part[w];
        norm[row] = (float)tot;
    }
}

constexpr uint32_t kRefineWarps = 8;

// One warp per (image, neuron).  Shared memory: kRefineWarps lists of T 16-bit transform indices.
__global__ void __launch_bounds__(kRefineWarps * 32)
refine_f32_kernel(const float* __restrict__ A, const float* __restrict__ anorm, uint32_t n, const float* __restrict__ B,
                  const float* __restrict__ bnorm, uint32_t T, uint32_t Kp, const float* __restrict__ est, float eps,
                  unsigned long long* __restrict__ keys, unsigned long long* __restrict__ stats)
{
    extern __shared__ uint16_t lists[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nn = blockIdx.x * kRefineWarps + warp, img = blockIdx.y;
    if (nn >= n) return;
    uint16_t* list = lists + (size_t)warp * T;
    const float* e = est + ((size_t)img * n + nn) * T;
    const float* nb = bnorm + (size_t)img * T;
    const float na = anorm[nn];

    const float4* a4 = reinterpret_cast<const float4*>(A + (size_t)nn * Kp);
    auto exact = [&](uint32_t t) {
        const float4* b4 = reinterpret_cast<const float4*>(B + ((size_t)img * T + t) * Kp);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
        for (uint32_t i = lane; i < Kp / 4; i += 32) {
            const float4 x = __ldg(a4 + i), y = __ldg(b4 + i);
            const float d0 = x.x - y.x, d1 = x.y - y.y, d2 = x.z - y.z, d3 = x.w - y.w;
            s0 = fmaf(d0, d0, s0); s1 = fmaf(d1, d1, s1); s2 = fmaf(d2, d2, s2); s3 = fmaf(d3, d3, s3);
        }
        float s = (s0 + s1) + (s2 + s3);
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        return s;                                         // the same value in every lane
    };

    // An upper limit of the true minimum: the smallest (estimate + its error bound), and the exact distance of the
    // transform with the smallest estimate.
    float ub = __int_as_float(0x7f800000);
    unsigned long long first = kKeyEmpty;                 // (estimate bits, transform) of the smallest estimate
    for (uint32_t t = lane; t < T; t += 32) {
        const float v = e[t];
        ub = fminf(ub, __fadd_rn(v, __fmul_rn(eps, __fadd_rn(na, nb[t]))));
        const unsigned long long k = ((unsigned long long)__float_as_uint(v) << 32) | t;
        first = k < first ? k : first;
    }
    for (int o = 16; o > 0; o >>= 1) {
        ub = fminf(ub, __shfl_xor_sync(0xffffffffu, ub, o));
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, first, o);
        first = other < first ? other : first;
    }
    const uint32_t t_first = (uint32_t)(first & 0xffffffffu);
    const float d_first = exact(t_first);
    ub = fminf(ub, d_first);

    // the other transforms whose true distance may be that small, in ascending order
    uint32_t count = 0;
    for (uint32_t t0 = 0; t0 < T; t0 += 32) {
        const uint32_t t = t0 + lane;
        const bool keep = t < T && t != t_first && __fsub_rn(e[t], __fmul_rn(eps, __fadd_rn(na, nb[t]))) <= ub;
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) list[count + __popc(m & ((1u << lane) - 1u))] = (uint16_t)t;
        count += __popc(m);
    }
    __syncwarp();

    // exact sums of squared differences for those; the first minimum wins (keys compare distance, then transform)
    unsigned long long best = ((unsigned long long)__float_as_uint(d_first) << 32) | t_first;
    float worst = fabsf(e[t_first] - d_first) / fmaxf(na + nb[t_first], 1e-30f);
    for (uint32_t c = 0; c < count; ++c) {
        const uint32_t t = list[c];
        const float s = exact(t);
        const unsigned long long key = ((unsigned long long)__float_as_uint(s) << 32) | t;
        best = key < best ? key : best;
        worst = fmaxf(worst, fabsf(e[t] - s) / fmaxf(na + nb[t], 1e-30f));
    }
    count += 1;                                           // the transform of the smallest estimate
    if (lane == 0) {
        keys[(size_t)img * n + nn] = best;
        if (stats) {
            atomicAdd(&stats[0], (unsigned long long)count);
            atomicMax(&stats[1], (unsigned long long)__float_as_uint(worst));     // non-negative floats order like their bits
        }
    }
}

} // namespace

cudaError_t launch_split_tf32(const float* src, uint64_t rows, uint32_t Kp, float* hi, float* lo, float* norm, cudaStream_t st)
{
    if (rows == 0) return cudaSuccess;
    if (Kp % 4 != 0 || rows > 0x7fffffffull) return cudaErrorInvalidValue;
    split_tf32_kernel<<<(unsigned)rows, kSplitThreads, 0, st>>>(src, Kp, hi, lo, norm);
    return cudaGetLastError();
}

cudaError_t launch_refine_f32(const Geometry& g, const float* A, const float* anorm, uint32_t n, const float* B, const float* bnorm,
                              uint32_t n_img, const float* est, float eps, unsigned long long* keys,
                              unsigned long long* stats, cudaStream_t st)
{
    if (n == 0 || n_img == 0) return cudaSuccess;
    const size_t smem = (size_t)kRefineWarps * g.T * sizeof(uint16_t);
    if (g.T > 65536u || smem > 200u * 1024u) return cudaErrorInvalidValue;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != attr_dev) {
        cudaError_t e = cudaFuncSetAttribute(refine_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    dim3 grid((n + kRefineWarps - 1) / kRefineWarps, n_img);
    refine_f32_kernel<<<grid, kRefineWarps * 32, smem, st>>>(A, anorm, n, B, bnorm, g.T, g.Kp, est, eps, keys, stats);
    return cudaGetLastError();
}

} // namespace pinkb
