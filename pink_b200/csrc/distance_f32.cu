// float32 distance kernel: direct differences on the FP32 pipe.
//
// Replaces euclidean_distance_kernel<bs, float, float> + second_step_kernel
// (src/CudaLib/euclidean_distance_kernel.h:61-102,
//  src/CudaLib/generate_euclidean_distance_matrix_second_step.h:18-38) for the
// float mode.  The Gram form is not used here: with d^2 << |n|^2 + |r|^2 its
// cancellation error exceeds the 1e-5 relative tolerance, so every term is
// (a - b)^2 accumulated with one FMA, k ascending.  Register-tiled like a
// GEMM: a CTA owns a BM x BN block of (neuron, transform) pairs, stages
// K slices of both operands in shared memory (k-major, so that a thread reads
// its TM neurons / TN transforms as float4), and each thread accumulates a
// TM x TN sub-block.  The epilogue keeps the first minimum over the thread's
// transforms per neuron, reduces across the threads sharing a neuron row with
// shuffles, and merges blocks with a 64-bit atomicMin on
// (float bits << 32 | transform); non-negative floats order like their bits.
#include "kernels.cuh"

namespace pinkb {

namespace {

constexpr int kBK = 16;

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
distance_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, uint32_t n, uint32_t T, uint32_t Kp,
                    unsigned long long* __restrict__ keys, float* __restrict__ s_out)
{
    constexpr int TX = BN / TN, TY = BM / TM, NT = TX * TY;
    __shared__ __align__(16) float As[2][kBK][BM + 4];
    __shared__ __align__(16) float Bs[2][kBK][BN + 4];

    const uint32_t img = blockIdx.z;
    const uint32_t m0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const float* Bi = B + (size_t)img * T * Kp;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    // Each row contributes kBK floats = 4 float4 per slice.
    constexpr int A_VEC = BM * kBK / 4, B_VEC = BN * kBK / 4;
    auto load_slice = [&](int buf, uint32_t k0) {
        for (int v = threadIdx.x; v < A_VEC; v += NT) {
            int r = v / (kBK / 4), c4 = v % (kBK / 4);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m0 + r < n) x = __ldg(reinterpret_cast<const float4*>(A + (size_t)(m0 + r) * Kp + k0) + c4);
            As[buf][c4 * 4 + 0][r] = x.x; As[buf][c4 * 4 + 1][r] = x.y;
            As[buf][c4 * 4 + 2][r] = x.z; As[buf][c4 * 4 + 3][r] = x.w;
        }
        for (int v = threadIdx.x; v < B_VEC; v += NT) {
            int r = v / (kBK / 4), c4 = v % (kBK / 4);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + r < T) x = __ldg(reinterpret_cast<const float4*>(Bi + (size_t)(t0 + r) * Kp + k0) + c4);
            Bs[buf][c4 * 4 + 0][r] = x.x; Bs[buf][c4 * 4 + 1][r] = x.y;
            Bs[buf][c4 * 4 + 2][r] = x.z; Bs[buf][c4 * 4 + 3][r] = x.w;
        }
    };

    const uint32_t nk = Kp / kBK;
    load_slice(0, 0);
    __syncthreads();
    for (uint32_t kb = 0; kb < nk; ++kb) {
        const int cur = kb & 1;
        if (kb + 1 < nk) load_slice(cur ^ 1, (kb + 1) * kBK);
#pragma unroll
        for (int k = 0; k < kBK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                float4 x = *reinterpret_cast<const float4*>(&As[cur][k][ty * TM + i]);
                a[i] = x.x; a[i + 1] = x.y; a[i + 2] = x.z; a[i + 3] = x.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                float4 x = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * TN + j]);
                b[j] = x.x; b[j + 1] = x.y; b[j + 2] = x.z; b[j + 3] = x.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    float d = a[i] - b[j];
                    acc[i][j] = fmaf(d, d, acc[i][j]);
                }
        }
        __syncthreads();
    }

    // First minimum over this thread's transforms, then across the TX threads of the row.
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const uint32_t nn = m0 + ty * TM + i;
        unsigned long long best = kKeyEmpty;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const uint32_t t = t0 + tx * TN + j;
            if (t < T) {
                unsigned long long key = ((unsigned long long)__float_as_uint(acc[i][j]) << 32) | t;
                best = key < best ? key : best;
                if (s_out && nn < n) s_out[((size_t)img * n + nn) * T + t] = acc[i][j];
            }
        }
#pragma unroll
        for (int o = TX / 2; o > 0; o >>= 1) {
            unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other < best ? other : best;
        }
        if (tx == 0 && nn < n && best != kKeyEmpty) atomicMin(&keys[(size_t)img * n + nn], best);
    }
}

} // namespace

cudaError_t launch_distance_f32(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why)
{
    const float* A = static_cast<const float*>(a.a0);
    const float* B = static_cast<const float*>(a.b0);
    float* s_out = static_cast<float*>(a.s_out);
    const uint64_t big = (uint64_t)((a.n + 127) / 128) * ((g.T + 127) / 128) * a.n_img;
    if (big >= 148) {
        dim3 grid((a.n + 127) / 128, (g.T + 127) / 128, a.n_img);
        distance_f32_kernel<128, 128, 8, 8><<<grid, 256, 0, st>>>(A, B, a.n, g.T, g.Kp, a.keys, s_out);
    } else {
        dim3 grid((a.n + 63) / 64, (g.T + 63) / 64, a.n_img);
        distance_f32_kernel<64, 64, 4, 4><<<grid, 256, 0, st>>>(A, B, a.n, g.T, g.Kp, a.keys, s_out);
    }
    *why = "distance_f32_kernel launch";
    return cudaGetLastError();
}

} // namespace pinkb
