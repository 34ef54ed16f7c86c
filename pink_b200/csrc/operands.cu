// Rotation-set generator and SOM operand quantiser.
//
// rotate_kernel replaces the reference's seven-launch sequence
//   thrust::fill + resize_kernel + rotate_bilinear_kernel + 3 x rotate_90_degrees_list
//   + flip_kernel              (src/CudaLib/generate_rotated_images.h:56-167, :170-294)
// followed by the per-image crop/convert of every transform
//   copy_and_transform_kernel  (src/CudaLib/copy_and_transform_kernel.h:15-29,
//                               src/CudaLib/generate_euclidean_distance_matrix.h:86-112)
// with ONE launch that never materialises the T x P float set: a CTA computes
// one interpolated base rotation (all channels) into shared memory, stores it
// once as float for the update step, and emits the distance operand rows of
// all eight transforms that are exact index permutations of that base (four
// quarter turns x optional flip) with packed, coalesced stores, plus each
// row's sum of squares.
//
// Arithmetic: every product and sum of the interpolation is rounded
// separately (__fmul_rn/__fadd_rn are never contracted to FMA), in the order
// of the reference's CPU code (src/ImageProcessingLib/rotate.h:31-63), so the
// float pixels are bit-identical to the CPU reference built without FMA.
#include "../../include/pink_b200.h"
#include "kernels.cuh"
#include "quant.cuh"

#include <atomic>
#include <type_traits>

#include <cmath>

namespace pinkb {

namespace {

// Centre crop / zero pad (src/CudaLib/resize_kernel.h:15-32, integer margins).
__device__ __forceinline__ float resize_pixel(const float* __restrict__ img, uint32_t id, uint32_t nd,
                                              uint32_t x, uint32_t y)
{
    if (id >= nd) {
        uint32_t m = (id - nd) / 2;
        return __ldg(img + (size_t)(x + m) * id + (y + m));
    }
    uint32_t m = (nd - id) / 2;
    if (x < m || y < m || x >= m + id || y >= m + id) return 0.0f;
    return __ldg(img + (size_t)(x - m) * id + (y - m));
}

template <typename Acc>
__device__ __forceinline__ Acc block_sum(Acc v, Acc* scratch)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    Acc r = 0;
    if (warp == 0) {
        r = lane < nw ? scratch[lane] : Acc(0);
        for (int o = 16; o > 0; o >>= 1) r += __shfl_down_sync(0xffffffffu, r, o);
    }
    return r;   // valid in thread 0
}

// Transform (flip f, quadrant j) reads pixel (x, y) from the base rotation at
// an affine position: flip is a row reversal applied last
// (src/CudaLib/flip_kernel.h:28); one quarter turn maps (x, y) <- (nd-1-y, x)
// (src/CudaLib/rotate_90_degrees_list.h:28).
constexpr int kRotThreads = 256;

// v / d for v * d < 2^32 with magic = floor(2^32 / d) + 1 (checked on the host).
// magic == 0 encodes the divisor 1.
__device__ __forceinline__ uint32_t fast_div(uint32_t v, uint32_t magic) { return magic ? __umulhi(v, magic) : v; }
inline uint32_t div_magic(uint32_t d) { return d == 1 ? 0u : (uint32_t)((1ull << 32) / d) + 1; }

template <int MODE> struct StageType;
template <> struct StageType<kModeU8>  { using type = uint8_t; };
template <> struct StageType<kModeU16> { using type = uint16_t; };
template <> struct StageType<kModeF32> { using type = float; };

template <int MODE>
__device__ __forceinline__ typename StageType<MODE>::type to_stage(float v)
{
    if (MODE == kModeU8) return (typename StageType<MODE>::type)quant_u8(v);
    if (MODE == kModeU16) return (typename StageType<MODE>::type)quant_u16(v);
    return (typename StageType<MODE>::type)v;
}

// One block = one base rotation of one image.
// Phase 1 walks the neuron-sized output row by row (a warp per row, lanes along
// the row) so that the row terms of the inverse rotation are computed once per
// row and the column terms once per thread; the float pixel goes to global
// memory (the update step reads it) and its converted value (uint8 / uint16 /
// float) is staged in shared memory -- for uint8 also transposed.
// Phase 2 emits, for each of the up to eight transforms that are index
// permutations of this base, the K-contiguous operand row, 16 elements per
// thread and store.  In uint8 mode a run of 16 operand bytes inside one row of
// the distance region is a contiguous (ascending or descending) run of bytes of
// the staged plane or of its transpose, so it is fetched with five aligned
// 32-bit loads and funnel shifts instead of sixteen byte gathers; sums of squares
// use dp4a on the packed bytes.
constexpr uint32_t kRotMaxSlots = 8;          // column slots (of 32) per thread with hoisted column terms
constexpr uint32_t kStagePad = 16;            // slack around the staged byte planes for aligned over-reads

// (five blocks per SM: the kernel lives on many resident warps; rarely taken paths may spill instead)
template <int MODE>
__global__ void __launch_bounds__(kRotThreads, 5)
rotate_kernel(Geometry g, const float* __restrict__ images, uint32_t use_smem, uint32_t magic_nd, uint32_t magic_ed,
              const float* __restrict__ cs, const float* __restrict__ sn, float* __restrict__ base_out,
              void* __restrict__ b0, void* __restrict__ b1, void* __restrict__ bnorm, uint32_t* __restrict__ rmax,
              void* __restrict__ b2)
{
    using stage_t = typename StageType<MODE>::type;
    extern __shared__ __align__(16) uint8_t rot_dyn[];
    // uint8: [pad | plane | pad | transposed plane | pad]; other modes: the plane only
    stage_t* stage = reinterpret_cast<stage_t*>(rot_dyn + (MODE == kModeU8 ? kStagePad : 0));
    uint8_t* stage_tr = rot_dyn + 2 * kStagePad + ((g.P + 15) & ~15u);
    __shared__ unsigned long long norm_s[8][kRotThreads / 32];   // per variant and warp: partial sum of squares
    __shared__ uint32_t vmax_s[kRotThreads / 32];
    uint32_t vmax = 0;                    // bit pattern of max |pixel| seen by this thread (NaN patterns compare highest)

    const uint32_t tq = blockIdx.x, img_i = blockIdx.y;
    const uint32_t nbase = g.q ? g.q : 1;
    const uint32_t P1 = g.nd * g.nd;
    const float* img = images + (size_t)img_i * g.C * g.id * g.id;
    float* gbase = base_out + ((size_t)img_i * nbase + tq) * g.P;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Phase 1: the base rotation (quadrant 0, no flip) of all channels.
    {
        const float sc = (g.id - 1) * 0.5f, dc = (g.nd - 1) * 0.5f, lim = (float)(g.id - 1);
        const float ca = tq ? cs[tq] : 1.0f, sa = tq ? sn[tq] : 0.0f;
        const uint32_t rows = g.C * g.nd;
        const uint32_t slots = (g.nd + 31) / 32;
        const bool hoisted = slots <= kRotMaxSlots;
        float pys[kRotMaxSlots], pyc[kRotMaxSlots];               // column terms py*sin, py*cos of this thread's columns
#pragma unroll
        for (uint32_t i = 0; i < kRotMaxSlots; ++i) {
            const float py = __fsub_rn((float)(lane + 32 * i), dc);
            pys[i] = __fmul_rn(py, sa);
            pyc[i] = __fmul_rn(py, ca);
        }
        const uint32_t idm1 = g.id - 1;
        // When the rotated neuron window lies strictly inside the image for every angle (half its diagonal, plus a
        // margin far above the rounding of the positions, within half the image), every source position s satisfies
        // 0 <= s < id - 1: none is out of range and no +1 tap falls outside, so the range test and the clamps below
        // are identities and are left out.
        const bool all_inside = __fadd_rn(__fmul_rn((float)(g.nd - 1), 0.70710678f), 0.01f) <= sc;
        for (uint32_t row = warp; row < rows; row += kRotThreads / 32) {
            const uint32_t c = fast_div(row, magic_nd), x = row - c * g.nd;
            const float* plane = img + (size_t)c * g.id * g.id;
            const float px = __fsub_rn((float)x, dc);
            const float xc = __fmul_rn(px, ca), xs = __fmul_rn(px, sa);
            const uint32_t row_idx = row * g.nd, tr_idx = c * P1 + x;
            // One output pixel; ys, yc are the column terms py*sin, py*cos.  Branch-free: positions
            // outside the image are clamped for the (then unused) taps and the result is zeroed.
            auto pixel = [&](uint32_t y, float ys, float yc) {
                float v;
                if (tq == 0) {                                     // block-uniform
                    v = resize_pixel(plane, g.id, g.nd, x, y);
                } else if (all_inside) {                           // uniform over the launch
                    const float sx = __fadd_rn(__fsub_rn(xc, ys), sc);
                    const float sy = __fadd_rn(__fadd_rn(xs, yc), sc);
                    const float tx = __fadd_rz(sx, 8388608.0f), ty = __fadd_rz(sy, 8388608.0f);
                    const uint32_t ix = __float_as_uint(tx) & 0x7FFFFFu, iy = __float_as_uint(ty) & 0x7FFFFFu;
                    const float rx = __fsub_rn(sx, __fsub_rn(tx, 8388608.0f));
                    const float ry = __fsub_rn(sy, __fsub_rn(ty, 8388608.0f));
                    const float cx = __fsub_rn(1.0f, rx), cy = __fsub_rn(1.0f, ry);
                    const float* r0 = plane + (ix * g.id + iy);
                    const float* r1 = r0 + g.id;
                    const float p00 = __ldg(r0), p01 = __ldg(r0 + 1), p10 = __ldg(r1), p11 = __ldg(r1 + 1);
                    const float t00 = __fmul_rn(__fmul_rn(cx, cy), p00);
                    const float t01 = __fmul_rn(__fmul_rn(cx, ry), p01);
                    const float t10 = __fmul_rn(__fmul_rn(rx, cy), p10);
                    const float t11 = __fmul_rn(__fmul_rn(rx, ry), p11);
                    v = __fadd_rn(__fadd_rn(__fadd_rn(t00, t01), t10), t11);
                } else {
                    // inverse rotation and bilinear taps; every product and sum rounded
                    // separately, in the order of src/ImageProcessingLib/rotate.h:37-63
                    const float sx = __fadd_rn(__fsub_rn(xc, ys), sc);
                    const float sy = __fadd_rn(__fadd_rn(xs, yc), sc);
                    const bool inside = fminf(sx, sy) >= 0.0f && fmaxf(sx, sy) <= lim;
                    const float qx = fminf(fmaxf(sx, 0.0f), lim), qy = fminf(fmaxf(sy, 0.0f), lim);   // = sx, sy when inside
                    // floor by adding 2^23 with truncation: exact for 0 <= s < 2^23, and it keeps
                    // the conversions off the (slow) conversion pipe
                    const float tx = __fadd_rz(qx, 8388608.0f), ty = __fadd_rz(qy, 8388608.0f);
                    const uint32_t ix = __float_as_uint(tx) & 0x7FFFFFu, iy = __float_as_uint(ty) & 0x7FFFFFu;
                    const float rx = __fsub_rn(qx, __fsub_rn(tx, 8388608.0f));
                    const float ry = __fsub_rn(qy, __fsub_rn(ty, 8388608.0f));
                    // the +1 taps carry weight 0 when they would fall outside; clamp the index
                    const uint32_t dx = ix < idm1 ? g.id : 0u, dy = iy < idm1 ? 1u : 0u;
                    const float cx = __fsub_rn(1.0f, rx), cy = __fsub_rn(1.0f, ry);
                    const uint32_t o00 = ix * g.id + iy;
                    const float p00 = __ldg(plane + o00), p01 = __ldg(plane + (o00 + dy));
                    const float p10 = __ldg(plane + (o00 + dx)), p11 = __ldg(plane + (o00 + dx + dy));
                    const float t00 = __fmul_rn(__fmul_rn(cx, cy), p00);
                    const float t01 = __fmul_rn(__fmul_rn(cx, ry), p01);
                    const float t10 = __fmul_rn(__fmul_rn(rx, cy), p10);
                    const float t11 = __fmul_rn(__fmul_rn(rx, ry), p11);
                    v = __fadd_rn(__fadd_rn(__fadd_rn(t00, t01), t10), t11);
                    v = inside ? v : 0.0f;
                }
                vmax = max(vmax, __float_as_uint(v) & 0x7FFFFFFFu);
                const uint32_t idx = row_idx + y;
                if (use_smem) {
                    const stage_t sv = to_stage<MODE>(v);
                    stage[idx] = sv;
                    if (MODE == kModeU8) stage_tr[tr_idx + y * g.nd] = (uint8_t)sv;
                }
                if (base_out) gbase[idx] = v;
            };
            if (hoisted) {
#pragma unroll
                for (uint32_t i = 0; i < kRotMaxSlots; ++i) {
                    const uint32_t y = lane + 32 * i;
                    if (y < g.nd) pixel(y, pys[i], pyc[i]);
                }
            } else {
                for (uint32_t y = lane; y < g.nd; y += 32) {
                    const float py = __fsub_rn((float)y, dc);
                    pixel(y, __fmul_rn(py, sa), __fmul_rn(py, ca));
                }
            }
        }
    }
    if (rmax) {
        vmax = __reduce_max_sync(0xffffffffu, vmax);
        if (lane == 0) vmax_s[warp] = vmax;
    }
    __syncthreads();   // also orders this block's global writes before its own reads below
    if (rmax && threadIdx.x == 0) {
        uint32_t m = 0;
        for (uint32_t wv = 0; wv < kRotThreads / 32; ++wv) m = max(m, vmax_s[wv]);
        atomicMax(rmax + img_i, m);
    }

    // Phase 2: operand rows of every transform derived from this base.
    const uint32_t nq = g.q ? 4 : 1, nv = nq * (g.flip ? 2 : 1);
    constexpr uint32_t kGroup = MODE == kModeF32 ? 4 : 16;         // operand elements per thread and store
    const uint32_t groups = (g.K + kGroup - 1) / kGroup;
    const int32_t nd = (int32_t)g.nd, nd1 = nd - 1;
    for (uint32_t v = 0; v < nv; ++v) {
        const uint32_t f = v / nq, j = v - f * nq;
        const uint32_t t = f * g.R + j * g.q + tq;
        const size_t orow = (size_t)img_i * g.T + t;
        int32_t ax, ay, a0;
        switch (j) {
            case 0:  ax = f ? -nd : nd; ay = 1;   a0 = f ? nd1 * nd : 0; break;
            case 1:  ax = f ? -1 : 1;   ay = -nd; a0 = nd1 * nd + (f ? nd1 : 0); break;
            case 2:  ax = f ? nd : -nd; ay = -1;  a0 = f ? nd1 : nd1 * nd + nd1; break;
            default: ax = f ? 1 : -1;   ay = nd;  a0 = f ? 0 : nd1; break;
        }
        a0 += (ax + ay) * (int32_t)g.off;            // x = off + i, y = off + jj
        const bool asc = j == 0 || j == 3;           // source bytes ascend with the operand index
        const uint8_t* run_plane = (j & 1) ? stage_tr : reinterpret_cast<const uint8_t*>(stage);
        // a thread's share of a row's sum of squares fits 32 bits in uint8 mode (K * 255^2 < 2^32)
        typename std::conditional<MODE == kModeU8, uint32_t, unsigned long long>::type acc = 0;
        float facc = 0.0f;                           // float mode with planes: this thread's share of the row's sum of squares
        for (uint32_t gi = threadIdx.x; gi < groups; gi += kRotThreads) {
            const uint32_t k = gi * kGroup;
            uint32_t r = fast_div(k, magic_ed), jj = k - r * g.ed;                  // r = c * ed + i
            uint32_t c = fast_div(r, magic_ed), i = r - c * g.ed;
            if (MODE == kModeU8 && use_smem && jj + 16 <= g.ed) {
                // whole group inside one row of the region: one contiguous run of 16 staged bytes
                const uint32_t x = g.off + i, sx = f ? (uint32_t)nd1 - x : x, y0 = g.off + jj;
                const uint32_t rowsel = j < 2 ? sx : (uint32_t)nd1 - sx;
                const uint32_t first = c * P1 + rowsel * g.nd + (asc ? y0 : (uint32_t)nd1 - y0 - 15u);
                const uint8_t* pa = run_plane + first;
                const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(pa) & 3u);
                const uint32_t* pw = reinterpret_cast<const uint32_t*>(pa - mis);
                uint32_t w[5], o[4];
#pragma unroll
                for (int m = 0; m < 5; ++m) w[m] = pw[m];
#pragma unroll
                for (int m = 0; m < 4; ++m) o[m] = __funnelshift_r(w[m], w[m + 1], mis * 8);
                if (!asc) {
                    const uint32_t r0 = __byte_perm(o[3], 0, 0x0123), r1 = __byte_perm(o[2], 0, 0x0123);
                    const uint32_t r2 = __byte_perm(o[1], 0, 0x0123), r3 = __byte_perm(o[0], 0, 0x0123);
                    o[0] = r0; o[1] = r1; o[2] = r2; o[3] = r3;
                }
                if (g.circle) {                              // zero the bytes outside the circle's span of this row
                    const ushort2 span = g.circle[i];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const int32_t c0 = (int32_t)jj + 4 * m;
                        const int32_t lo = min(max((int32_t)span.x - c0, 0), 4), hi = min(max((int32_t)span.y - c0, 0), 4);
                        uint32_t keep = 0;
                        if (hi > lo) keep = (hi == 4 ? 0xFFFFFFFFu : (1u << (8 * hi)) - 1u) & ~((1u << (8 * lo)) - 1u);
                        o[m] &= keep;
                    }
                }
#pragma unroll
                for (int m = 0; m < 4; ++m) acc = __dp4a(o[m], o[m], (uint32_t)acc);
                reinterpret_cast<uint4*>(static_cast<uint8_t*>(b0) + orow * g.Kp)[gi] = make_uint4(o[0], o[1], o[2], o[3]);
                continue;
            }
            int32_t s = (int32_t)(c * P1) + ax * (int32_t)i + ay * (int32_t)jj + a0;
            stage_t val[kGroup];
#pragma unroll
            for (uint32_t e = 0; e < kGroup; ++e) {
                val[e] = 0;
                if (k + e < g.K && in_region(g, i, jj)) val[e] = use_smem ? stage[s] : to_stage<MODE>(gbase[s]);
                ++jj; s += ay;
                if (jj == g.ed) {
                    jj = 0; ++i;
                    if (i == g.ed) { i = 0; ++c; }
                    s = (int32_t)(c * P1) + ax * (int32_t)i + a0;
                }
            }
            if (MODE == kModeU8) {
                uint32_t wv[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    wv[q4] = (uint32_t)val[4 * q4] | ((uint32_t)val[4 * q4 + 1] << 8)
                           | ((uint32_t)val[4 * q4 + 2] << 16) | ((uint32_t)val[4 * q4 + 3] << 24);
                    acc = __dp4a(wv[q4], wv[q4], (uint32_t)acc);
                }
                reinterpret_cast<uint4*>(static_cast<uint8_t*>(b0) + orow * g.Kp)[gi] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            } else if (MODE == kModeU16) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    hi[q4] = lo[q4] = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t qv = (uint32_t)val[4 * q4 + e];
                        hi[q4] |= (qv >> 8) << (8 * e);
                        lo[q4] |= (qv & 255u) << (8 * e);
                        acc += (unsigned long long)qv * qv;
                    }
                }
                reinterpret_cast<uint4*>(static_cast<uint8_t*>(b0) + orow * g.Kp)[gi] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                reinterpret_cast<uint4*>(static_cast<uint8_t*>(b1) + orow * g.Kp)[gi] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            } else {
                const float4 v4 = make_float4((float)val[0], (float)val[1], (float)val[2], (float)val[3]);
                reinterpret_cast<float4*>(static_cast<float*>(b0) + orow * g.Kp)[gi] = v4;
                if (b1) {
                    // planes of the tensor-core estimate: the top 19 bits of every value and the (exact) rest
                    float4 h, l;
                    h.x = __uint_as_float(__float_as_uint(v4.x) & 0xFFFFE000u); l.x = __fsub_rn(v4.x, h.x);
                    h.y = __uint_as_float(__float_as_uint(v4.y) & 0xFFFFE000u); l.y = __fsub_rn(v4.y, h.y);
                    h.z = __uint_as_float(__float_as_uint(v4.z) & 0xFFFFE000u); l.z = __fsub_rn(v4.z, h.z);
                    h.w = __uint_as_float(__float_as_uint(v4.w) & 0xFFFFE000u); l.w = __fsub_rn(v4.w, h.w);
                    reinterpret_cast<float4*>(static_cast<float*>(b1) + orow * g.Kp)[gi] = h;
                    reinterpret_cast<float4*>(static_cast<float*>(b2) + orow * g.Kp)[gi] = l;
                    facc += (v4.x * v4.x + v4.y * v4.y) + (v4.z * v4.z + v4.w * v4.w);
                }
            }
        }
        if (MODE != kModeF32) {
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
            if (lane == 0) norm_s[v][warp] = acc;
        } else if (b1) {
            for (int o = 16; o > 0; o >>= 1) facc += __shfl_down_sync(0xffffffffu, facc, o);
            if (lane == 0) norm_s[v][warp] = (unsigned long long)__double_as_longlong((double)facc);
        }
    }
    if (MODE != kModeF32 || b1) {
        __syncthreads();
        if (threadIdx.x < nv) {
            const uint32_t v = threadIdx.x, f = v / nq, j = v - f * nq;
            const size_t orow = (size_t)img_i * g.T + f * g.R + j * g.q + tq;
            if (MODE == kModeF32) {
                double tot = 0.0;
                for (uint32_t wv = 0; wv < kRotThreads / 32; ++wv) tot += __longlong_as_double((long long)norm_s[v][wv]);
                static_cast<float*>(bnorm)[orow] = (float)tot;
            } else {
                unsigned long long tot = 0;
                for (uint32_t wv = 0; wv < kRotThreads / 32; ++wv) tot += norm_s[v][wv];
                if (MODE == kModeU8) static_cast<uint32_t*>(bnorm)[orow] = (uint32_t)tot;
                else static_cast<unsigned long long*>(bnorm)[orow] = tot;
            }
        }
    }
}

// One CTA per neuron: centre crop of every channel, convert, row sum of squares.
// Replaces the per-image copy_and_transform_kernel pass over the whole SOM
// (src/CudaLib/generate_euclidean_distance_matrix.h:64-84); here it runs once
// when a SOM is loaded, afterwards the update kernel refreshes the rows it changes.
template <int MODE>
__global__ void __launch_bounds__(256)
quantize_som_kernel(Geometry g, const float* __restrict__ som, void* __restrict__ a0, void* __restrict__ a1,
                    void* __restrict__ anorm, uint2* __restrict__ wrange)
{
    __shared__ unsigned long long red[8];
    __shared__ uint32_t lo_s[8], hi_s[8];
    const size_t n = blockIdx.x;
    const float* src = som + n * g.Pp;
    const uint32_t P1 = g.nd * g.nd, K1 = g.ed * g.ed;
    const uint32_t groups = (g.K + 3) / 4;
    unsigned long long acc = 0;
    for (uint32_t k4 = threadIdx.x; k4 < groups; k4 += blockDim.x) {
        float val[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            uint32_t k = k4 * 4 + e;
            val[e] = 0.0f;
            if (k < g.K) {
                uint32_t c = k / K1, r = k - c * K1;
                uint32_t i = r / g.ed, jj = r - i * g.ed;
                if (in_region(g, i, jj)) val[e] = src[c * P1 + (g.off + i) * g.nd + g.off + jj];
            }
        }
        if (MODE == kModeU8) {
            uint32_t q0 = quant_u8(val[0]), q1 = quant_u8(val[1]), q2 = quant_u8(val[2]), q3 = quant_u8(val[3]);
            acc += q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3;
            reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a0) + n * g.Kp)[k4] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
        } else if (MODE == kModeU16) {
            uint32_t q0 = quant_u16(val[0]), q1 = quant_u16(val[1]), q2 = quant_u16(val[2]), q3 = quant_u16(val[3]);
            acc += (unsigned long long)q0 * q0 + (unsigned long long)q1 * q1
                 + (unsigned long long)q2 * q2 + (unsigned long long)q3 * q3;
            reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a0) + n * g.Kp)[k4] =
                (q0 >> 8) | ((q1 >> 8) << 8) | ((q2 >> 8) << 16) | ((q3 >> 8) << 24);
            reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a1) + n * g.Kp)[k4] =
                (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) | ((q3 & 255) << 24);
        } else {
            reinterpret_cast<float4*>(static_cast<float*>(a0) + n * g.Kp)[k4] = make_float4(val[0], val[1], val[2], val[3]);
        }
    }
    if (MODE != kModeF32) {
        unsigned long long s = block_sum<unsigned long long>(acc, red);
        if (threadIdx.x == 0) {
            if (MODE == kModeU8) static_cast<uint32_t*>(anorm)[n] = (uint32_t)s;
            else static_cast<unsigned long long*>(anorm)[n] = s;
        }
    }
    if (wrange) {
        // bit patterns of min |w| and max |w| over the whole neuron (integer order = float order for
        // non-negative values; NaN patterns compare highest)
        uint32_t lo = 0xFFFFFFFFu, hi = 0;
        for (uint32_t i = threadIdx.x; i < g.P; i += blockDim.x) {
            const uint32_t b = __float_as_uint(src[i]) & 0x7FFFFFFFu;
            lo = min(lo, b); hi = max(hi, b);
        }
        lo = __reduce_min_sync(0xffffffffu, lo); hi = __reduce_max_sync(0xffffffffu, hi);
        if ((threadIdx.x & 31) == 0) { lo_s[threadIdx.x >> 5] = lo; hi_s[threadIdx.x >> 5] = hi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint32_t wv = 1; wv < blockDim.x / 32; ++wv) { lo = min(lo, lo_s[wv]); hi = max(hi, hi_s[wv]); }
            wrange[n] = make_uint2(lo, hi);
        }
    }
}

__global__ void fill_keys_kernel(unsigned long long* keys, size_t count)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        keys[i] = kKeyEmpty;
}

constexpr size_t kRotateSmemLimit = 200 * 1024;

template <int MODE>
cudaError_t rotate_dispatch(const Geometry& g, const float* images, uint32_t n_img, const float* cs, const float* sn,
                     float* base_out, void* b0, void* b1, void* bnorm, cudaStream_t st, uint32_t* rmax, void* b2)
{
    size_t smem = MODE == kModeU8 ? 2 * (((size_t)g.P + 15) & ~size_t(15)) + 3 * kStagePad
                                  : (size_t)g.P * sizeof(typename StageType<MODE>::type);
    uint32_t use_smem = smem <= kRotateSmemLimit;
    if (!use_smem) smem = 0;
    // Dynamic shared memory above 48 KB is an opt-in, per-device function attribute.
    static thread_local int attr_dev = -1;
    static thread_local size_t attr_bytes = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev != attr_dev || smem > attr_bytes)) {
        cudaError_t e = cudaFuncSetAttribute(rotate_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
        attr_bytes = smem;
    }
    if ((uint64_t)g.P * g.nd >= (1ull << 32) || (uint64_t)g.K * g.ed >= (1ull << 32)) return cudaErrorInvalidValue;
    const uint32_t magic_nd = div_magic(g.nd), magic_ed = div_magic(g.ed);
    dim3 grid(g.q ? g.q : 1, n_img);
    rotate_kernel<MODE><<<grid, kRotThreads, smem, st>>>(g, images, use_smem, magic_nd, magic_ed, cs, sn, base_out,
                                                         b0, b1, bnorm, rmax, b2);
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_rotate(const Geometry& g, const float* images, uint32_t n_img, const float* cs, const float* sn,
                          float* base_out, void* b0, void* b1, void* bnorm, cudaStream_t st, uint32_t* rmax, void* b2)
{
    if (n_img == 0) return cudaSuccess;
    if (g.mode == kModeU8) return rotate_dispatch<kModeU8>(g, images, n_img, cs, sn, base_out, b0, b1, bnorm, st, rmax, nullptr);
    if (g.mode == kModeU16) return rotate_dispatch<kModeU16>(g, images, n_img, cs, sn, base_out, b0, b1, bnorm, st, rmax, nullptr);
    // float: the planes are written only when both are given (b1 alone has no meaning in this mode)
    return rotate_dispatch<kModeF32>(g, images, n_img, cs, sn, base_out, b0, b2 ? b1 : nullptr, bnorm, st, rmax, b2);
}

cudaError_t launch_quantize_som(const Geometry& g, const float* som, uint32_t n, void* a0, void* a1, void* anorm,
                                cudaStream_t st, uint2* wrange)
{
    if (n == 0) return cudaSuccess;
    if (g.mode == kModeU8) quantize_som_kernel<kModeU8><<<n, 256, 0, st>>>(g, som, a0, a1, anorm, wrange);
    else if (g.mode == kModeU16) quantize_som_kernel<kModeU16><<<n, 256, 0, st>>>(g, som, a0, a1, anorm, wrange);
    else quantize_som_kernel<kModeF32><<<n, 256, 0, st>>>(g, som, a0, a1, anorm, wrange);
    return cudaGetLastError();
}

cudaError_t launch_fill_keys(unsigned long long* keys, size_t count, cudaStream_t st)
{
    if (count == 0) return cudaSuccess;
    unsigned blocks = (unsigned)((count + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    fill_keys_kernel<<<blocks, 256, 0, st>>>(keys, count);
    return cudaGetLastError();
}

} // namespace pinkb

// ---------------------------------------------------------------------------
// Rotation-set entry point that never allocates.
//
// pink_b200_op_rotate stages the cos/sin table of the rotation angles in device
// memory it obtains with cudaMalloc on every call.  Some callers must not do
// that: code running while the CUDA allocator is locked or forbidden (inside a
// memory-pool or caching-allocator callback, in a process whose device memory
// is fully pre-reserved by its own arena, or in a latency-critical loop where an
// implicit device synchronisation of cudaMalloc/cudaFree is unacceptable).
// For them the table lives in the fixed device array below, which every GPU
// that loads this library holds until the process exits.
namespace pinkb {
namespace {

constexpr uint32_t kStaticMaxQuadrant = 4096;     // rotations per quadrant, i.e. number_of_rotations <= 16384
static __device__ __align__(256) float g_rotate_scratch[2 * kStaticMaxQuadrant];   // [cos | sin], 32 KB

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t rotate_scratch_address(float** out)
{
    constexpr int kMaxDevices = 64;
    static std::atomic<float*> addr[kMaxDevices];        // first calls may come from several host threads
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    float* known = addr[dev].load(std::memory_order_acquire);
    if (!known) {
        // In host code the array's name is only a handle; the kernels need its device address.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_rotate_scratch);
        if (e != cudaSuccess) return e;
        known = static_cast<float*>(p);
        addr[dev].store(known, std::memory_order_release);   // every thread looks up the same address
    }
    *out = known;
    return cudaSuccess;
}

} // namespace
} // namespace pinkb

extern "C" int pink_b200_op_rotate_static(const pink_b200_config* cfg, const float* dev_images, uint32_t n_img,
                                          float* dev_base, void* dev_b0, void* dev_b1, void* dev_bnorm, void* stream)
{
    using namespace pinkb;
    if (!cfg || !dev_images || !dev_b0) return report_error(PINK_B200_EINVAL, "null argument");
    Geometry g{};
    int rc = geometry_from_config(cfg, &g);
    if (rc) return rc;
    const uint32_t nq = g.q ? g.q : 1;
    if (nq > kStaticMaxQuadrant)
        return report_error(PINK_B200_EINVAL,
                            "pink_b200_op_rotate_static supports at most 16384 rotations (4096 per quadrant); "
                            "use pink_b200_op_rotate for more");
    if (!dev_base && (size_t)g.P * sizeof(float) > kRotateSmemLimit)
        return report_error(PINK_B200_EINVAL, "dev_base is required when a base rotation does not fit shared memory");
    float* scratch = nullptr;
    cudaError_t e = rotate_scratch_address(&scratch);
    if (e != cudaSuccess) return report_error(PINK_B200_ECUDA, cudaGetErrorString(e));

    // cos/sin of t * (float(2*pi)/R), t < R/4, with the reference's expressions
    // (src/SelfOrganizingMapLib/generate_rotated_images.h:70, src/ImageProcessingLib/rotate.h:20-21).
    static thread_local float table[2 * kStaticMaxQuadrant];
    const float step = static_cast<float>(2 * M_PI) / g.R;
    for (uint32_t t = 0; t < nq; ++t) {
        const float angle = t * step;
        table[t] = std::cos(angle);
        table[nq + t] = std::sin(angle);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The shared array still holds the previous call's table; the part this call uses is overwritten in full.
    e = cudaMemcpyAsync(scratch, table, 2 * nq * sizeof(float), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = launch_rotate(g, dev_images, n_img, scratch, scratch + nq, dev_base, dev_b0, dev_b1, dev_bnorm, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);      // `table` is reused by this thread's next call
    if (e != cudaSuccess) return report_error(PINK_B200_ECUDA, cudaGetErrorString(e));
    return PINK_B200_OK;
}
