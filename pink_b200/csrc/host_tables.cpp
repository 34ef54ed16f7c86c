// Host-side tables that feed the device path: SOM grid distances and the
// N x N update-factor table.  The reference builds the same table in the
// TrainerCommon constructor (src/SelfOrganizingMapLib/Trainer.h:69-76) from
// layout.get_distance (CartesianLayout.h:47-60,108-114; HexagonalLayout.h:90-118)
// and a distribution functor (src/UtilitiesLib/DistributionFunctor.cpp:18-59).
// All arithmetic is float32 with the reference's expression shapes so that the
// factors, and therefore the trained weights, agree bit for bit.
#include "../../include/pink_b200.h"

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <vector>

namespace {

struct Cell { int32_t q, r; };

// Axial position of array index i in the row-packed hexagon of side `dim`.
Cell hex_cell(uint32_t i, const std::vector<uint32_t>& row_offset, uint32_t radius)
{
    uint32_t r = 0;
    while (i >= row_offset[r + 1]) ++r;
    uint32_t q = i - row_offset[r];
    if (radius > r) q += radius - r;
    return { (int32_t)q, (int32_t)r };
}

float neighbourhood(uint32_t func, float d, float p0, float p1)
{
    switch (func) {
        case PINK_B200_FUNC_GAUSSIAN:
            return p1 / (p0 * std::sqrt(2.0f * static_cast<float>(M_PI))) * std::exp(-0.5f * std::pow(d / p0, 2.0f));
        case PINK_B200_FUNC_UNITY_GAUSSIAN:
            return p1 * std::exp(-0.5f * std::pow(d / p0, 2.0f));
        case PINK_B200_FUNC_MEXICAN_HAT: {
            const float d2 = d * d, s2 = p0 * p0;
            return 2.0f * p1 / (std::sqrt(3.0f * p0) * std::pow(static_cast<float>(M_PI), 0.25f))
                   * (1.0f - d2 / s2) * std::exp(-d2 / (2.0f * s2));
        }
        default:
            return d <= p0 ? 1.0f : 0.0f;
    }
}

} // namespace

extern "C" {

int pink_b200_shard_range(uint32_t n_neurons, uint32_t world_size, uint32_t rank, uint32_t* first, uint32_t* count)
{
    if (world_size == 0 || rank >= world_size || world_size > n_neurons || !first || !count) return PINK_B200_EINVAL;
    const uint32_t base = n_neurons / world_size, extra = n_neurons % world_size;
    *count = base + (rank < extra ? 1 : 0);
    *first = rank * base + (rank < extra ? rank : extra);
    return PINK_B200_OK;
}

uint32_t pink_b200_som_size(uint32_t som_layout, uint32_t dim0, uint32_t dim1)
{
    if (som_layout == PINK_B200_LAYOUT_CARTESIAN) return dim0 * dim1;
    const uint32_t radius = (dim0 - 1) / 2;
    return dim0 * dim0 - radius * (radius + 1);
}

int pink_b200_som_distances(uint32_t som_layout, uint32_t dim0, uint32_t dim1, float* out)
{
    if (!out || dim0 == 0 || dim1 == 0) return PINK_B200_EINVAL;
    const uint32_t N = pink_b200_som_size(som_layout, dim0, dim1);
    if (som_layout == PINK_B200_LAYOUT_CARTESIAN) {
        for (uint32_t i = 0; i < N; ++i)
            for (uint32_t j = 0; j < N; ++j) {
                const uint32_t a[2] = { i % dim1, i / dim1 }, b[2] = { j % dim1, j / dim1 };
                float d = 0.0f;
                for (int k = 0; k < 2; ++k) {
                    const float diff = static_cast<float>(a[k]) - static_cast<float>(b[k]);
                    d += static_cast<float>(static_cast<double>(diff) * static_cast<double>(diff));
                }
                out[(size_t)i * N + j] = std::sqrt(d);
            }
        return PINK_B200_OK;
    }
    if (som_layout != PINK_B200_LAYOUT_HEXAGONAL || dim0 % 2 == 0 || dim0 != dim1) return PINK_B200_EINVAL;
    const uint32_t radius = (dim0 - 1) / 2;
    std::vector<uint32_t> row_offset(dim0 + 1, 0);
    for (uint32_t r = 0; r < dim0; ++r)
        row_offset[r + 1] = row_offset[r] + dim0 - (r > radius ? r - radius : radius - r);
    std::vector<Cell> cells(N);
    for (uint32_t i = 0; i < N; ++i) cells[i] = hex_cell(i, row_offset, radius);
    for (uint32_t i = 0; i < N; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            const int32_t dx = cells[i].q - cells[j].q, dy = cells[i].r - cells[j].r;
            const int32_t hops = ((dx >= 0) == (dy >= 0)) ? std::abs(dx + dy) : std::max(std::abs(dx), std::abs(dy));
            out[(size_t)i * N + j] = static_cast<float>(hops);
        }
    return PINK_B200_OK;
}

int pink_b200_som_distances_3d(uint32_t dim0, uint32_t dim1, uint32_t dim2, float* out)
{
    if (!out || dim0 == 0 || dim1 == 0 || dim2 == 0) return PINK_B200_EINVAL;
    const uint32_t N = dim0 * dim1 * dim2;
    // the reference's position of an array index, expression by expression
    auto cell = [&](uint32_t i, uint32_t p[3]) {
        p[2] = i / dim0 / dim1;
        p[1] = (i - p[2] * dim0 * dim1) / dim1;
        p[0] = i % dim1;
    };
    for (uint32_t i = 0; i < N; ++i)
        for (uint32_t j = 0; j < N; ++j) {
            uint32_t a[3], b[3];
            cell(i, a);
            cell(j, b);
            float d = 0.0f;
            for (int k = 0; k < 3; ++k) {
                const float diff = static_cast<float>(a[k]) - static_cast<float>(b[k]);
                d += static_cast<float>(static_cast<double>(diff) * static_cast<double>(diff));
            }
            out[(size_t)i * N + j] = std::sqrt(d);
        }
    return PINK_B200_OK;
}

// ---- update factors per distance class ------------------------------------------------------------------------
// The map distance of two neurons takes few distinct values: it depends only on the absolute coordinate differences
// (cartesian) or is the hop count (hexagonal).  A class index enumerates them; coordinates and classes follow the
// reference's index -> position expressions above, so that lut[class(i, j)] == function(get_distance(i, j)) bit for bit.

static bool layout_ok(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2)
{
    if (dim0 == 0 || dim1 == 0 || dim2 == 0) return false;
    if (som_layout == PINK_B200_LAYOUT_CARTESIAN) return true;
    return som_layout == PINK_B200_LAYOUT_HEXAGONAL && dim2 == 1 && dim0 % 2 == 1 && dim0 == dim1;
}

uint32_t pink_b200_distance_classes(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, float* distances,
                                    uint32_t capacity)
{
    if (!layout_ok(som_layout, dim0, dim1, dim2)) return 0;
    if (som_layout == PINK_B200_LAYOUT_HEXAGONAL) {
        const uint32_t n = dim0;                       // hop counts 0 .. 2 * radius
        if (distances) for (uint32_t h = 0; h < n && h < capacity; ++h) distances[h] = static_cast<float>(h);
        return n;
    }
    const uint64_t n64 = (uint64_t)dim0 * dim1 * dim2;
    if (n64 > 0xFFFFFFFFull) return 0;
    if (distances) {
        // class (|d2| * dim0 + |d1|) * dim1 + |d0|; the sum runs over the coordinates in the reference's order
        uint32_t c = 0;
        for (uint32_t d2 = 0; d2 < dim2; ++d2)
            for (uint32_t d1 = 0; d1 < dim0; ++d1)
                for (uint32_t d0 = 0; d0 < dim1; ++d0, ++c) {
                    if (c >= capacity) continue;
                    const float diff[3] = { static_cast<float>(d0), static_cast<float>(d1), static_cast<float>(d2) };
                    float d = 0.0f;
                    for (int k = 0; k < (dim2 > 1 ? 3 : 2); ++k)
                        d += static_cast<float>(static_cast<double>(diff[k]) * static_cast<double>(diff[k]));
                    distances[c] = std::sqrt(d);
                }
    }
    return (uint32_t)n64;
}

int pink_b200_som_coordinates(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, int16_t* out)
{
    if (!out || !layout_ok(som_layout, dim0, dim1, dim2)) return PINK_B200_EINVAL;
    if (dim0 > 32767 || dim1 > 32767 || dim2 > 32767) return PINK_B200_EINVAL;
    if (som_layout == PINK_B200_LAYOUT_HEXAGONAL) {
        const uint32_t N = pink_b200_som_size(som_layout, dim0, dim1), radius = (dim0 - 1) / 2;
        std::vector<uint32_t> row_offset(dim0 + 1, 0);
        for (uint32_t r = 0; r < dim0; ++r)
            row_offset[r + 1] = row_offset[r] + dim0 - (r > radius ? r - radius : radius - r);
        for (uint32_t i = 0; i < N; ++i) {
            const Cell c = hex_cell(i, row_offset, radius);
            out[4 * i] = (int16_t)c.q; out[4 * i + 1] = (int16_t)c.r; out[4 * i + 2] = 0; out[4 * i + 3] = 0;
        }
        return PINK_B200_OK;
    }
    const uint32_t N = dim0 * dim1 * dim2;
    for (uint32_t i = 0; i < N; ++i) {
        uint32_t p[3];
        if (dim2 > 1) { p[2] = i / dim0 / dim1; p[1] = (i - p[2] * dim0 * dim1) / dim1; p[0] = i % dim1; }
        else { p[0] = i % dim1; p[1] = i / dim1; p[2] = 0; }
        out[4 * i] = (int16_t)p[0]; out[4 * i + 1] = (int16_t)p[1]; out[4 * i + 2] = (int16_t)p[2]; out[4 * i + 3] = 0;
    }
    return PINK_B200_OK;
}

int pink_b200_update_lut(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t func, float p0, float p1,
                         float max_update_distance, float* lut, uint32_t capacity)
{
    if (!lut || func > PINK_B200_FUNC_STEP) return PINK_B200_EINVAL;
    if (func == PINK_B200_FUNC_MEXICAN_HAT && p0 <= 0.0f) return PINK_B200_EINVAL;
    const uint32_t n = pink_b200_distance_classes(som_layout, dim0, dim1, dim2, nullptr, 0);
    if (n == 0 || n > capacity) return PINK_B200_EINVAL;
    pink_b200_distance_classes(som_layout, dim0, dim1, dim2, lut, n);
    for (uint32_t c = 0; c < n; ++c) {
        const float d = lut[c];
        lut[c] = (max_update_distance <= 0.0f || d < max_update_distance) ? neighbourhood(func, d, p0, p1) : 0.0f;
    }
    return PINK_B200_OK;
}

static int apply_neighbourhood(size_t count, uint32_t func, float p0, float p1, float max_update_distance, float* out)
{
    for (size_t i = 0; i < count; ++i) {
        const float d = out[i];
        out[i] = (max_update_distance <= 0.0f || d < max_update_distance) ? neighbourhood(func, d, p0, p1) : 0.0f;
    }
    return PINK_B200_OK;
}

int pink_b200_update_factors_3d(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t func, float p0, float p1,
                                float max_update_distance, float* out)
{
    if (func > PINK_B200_FUNC_STEP) return PINK_B200_EINVAL;
    if (func == PINK_B200_FUNC_MEXICAN_HAT && p0 <= 0.0f) return PINK_B200_EINVAL;
    int rc = pink_b200_som_distances_3d(dim0, dim1, dim2, out);
    if (rc) return rc;
    const size_t N = (size_t)dim0 * dim1 * dim2;
    return apply_neighbourhood(N * N, func, p0, p1, max_update_distance, out);
}

int pink_b200_update_factors(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t func, float p0, float p1,
                             float max_update_distance, float* out)
{
    if (func > PINK_B200_FUNC_STEP) return PINK_B200_EINVAL;
    if (func == PINK_B200_FUNC_MEXICAN_HAT && p0 <= 0.0f) return PINK_B200_EINVAL;
    int rc = pink_b200_som_distances(som_layout, dim0, dim1, out);
    if (rc) return rc;
    const size_t N = pink_b200_som_size(som_layout, dim0, dim1);
    return apply_neighbourhood(N * N, func, p0, p1, max_update_distance, out);
}

} // extern "C"
