// ref_shim.cpp -- thin extern "C" window onto the UNMODIFIED reference CPU
// implementation (PINK's header templates), compiled in place from the
// reference source tree into oracle/_ref/libpink_ref.so by oracle/Makefile.
//
// TEST INFRASTRUCTURE ONLY: used to validate the CPU restatement in
// pink_oracle.c, to generate the golden fixtures under tests/golden/, and as
// the timed CPU baseline of the benchmark's reference arm.  The shipped
// library never links or loads it.  No reference source is copied here; the
// shim only instantiates and calls the reference's public templates:
//   SpatialTransformer      src/SelfOrganizingMapLib/generate_rotated_images.h
//   Trainer<...,false>      src/SelfOrganizingMapLib/Trainer.h:119-193
//   Mapper<...,false>       src/SelfOrganizingMapLib/Mapper.h:93-123
//   layouts / functors      CartesianLayout.h, HexagonalLayout.h,
//                           src/UtilitiesLib/DistributionFunctor.h, Filler.h
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <sstream>
#include <vector>
#include <omp.h>

#include "SelfOrganizingMapLib/CartesianLayout.h"
#include "SelfOrganizingMapLib/HexagonalLayout.h"
#include "SelfOrganizingMapLib/Data.h"
#include "SelfOrganizingMapLib/SOM.h"
#include "SelfOrganizingMapLib/DataIteratorShuffled.h"
#include "SelfOrganizingMapLib/Trainer.h"
#include "SelfOrganizingMapLib/Mapper.h"
#include "SelfOrganizingMapLib/generate_rotated_images.h"
#include "UtilitiesLib/DistributionFunctor.h"
#include "UtilitiesLib/Filler.h"

using namespace pink;

namespace {

std::function<float(float)> make_func(int func, float p0, float p1)
{
    switch (func) {
        case 0: return GaussianFunctor(p0, p1);
        case 1: return UnityGaussianFunctor(p0, p1);
        case 2: return MexicanHatFunctor(p0, p1);
        default: return StepFunctor(p0);
    }
}

template <typename L> L make_som_layout(uint32_t d0, uint32_t d1);
template <> CartesianLayout<2> make_som_layout(uint32_t d0, uint32_t d1) { return CartesianLayout<2>{{d0, d1}}; }
template <> HexagonalLayout make_som_layout(uint32_t d0, uint32_t) { return HexagonalLayout({d0, d0}); }

template <typename L> L make_data_layout(uint32_t c, uint32_t d);
template <> CartesianLayout<2> make_data_layout(uint32_t, uint32_t d) { return CartesianLayout<2>{{d, d}}; }
template <> CartesianLayout<3> make_data_layout(uint32_t c, uint32_t d) { return CartesianLayout<3>{{c, d, d}}; }

// A persistent trainer so that many images can be pushed through one
// Trainer object, as the reference's CLI loop does.
struct Session
{
    virtual ~Session() {}
    virtual void train(const float* img) = 0;
    virtual void map(const float* img, float* dist, uint32_t* rot) = 0;
    virtual float* som_data() = 0;
    virtual size_t som_size() = 0;
    virtual void counts(uint32_t* out) = 0;
};

template <typename SL, typename DL>
struct SessionT : Session
{
    typedef SOM<SL, DL, float> SOMT;
    SOMT som;
    DL img_layout;
    std::unique_ptr<Trainer<SL, DL, float, false>> trainer;
    std::unique_ptr<Mapper<SL, DL, float, false>> mapper;

    SessionT(const float* som_in, uint32_t s0, uint32_t s1, uint32_t C, uint32_t id, uint32_t nd, uint32_t ed,
             uint32_t R, bool flip, int func, float p0, float p1, float max_dist, bool for_map, int shape)
     : som(make_som_layout<SL>(s0, s1), make_data_layout<DL>(C, nd)),
       img_layout(make_data_layout<DL>(C, id))
    {
        std::memcpy(som.get_data_pointer(), som_in, som.size() * sizeof(float));
        if (for_map)
            mapper.reset(new Mapper<SL, DL, float, false>(som, 0, R, flip, Interpolation::BILINEAR, ed,
                shape ? EuclideanDistanceShape::CIRCULAR : EuclideanDistanceShape::QUADRATIC));
        else
            trainer.reset(new Trainer<SL, DL, float, false>(som, make_func(func, p0, p1), 0, R, flip, max_dist,
                Interpolation::BILINEAR, ed, shape ? EuclideanDistanceShape::CIRCULAR : EuclideanDistanceShape::QUADRATIC));
    }
    void train(const float* img) override
    {
        Data<DL, float> d(img_layout, std::vector<float>(img, img + img_layout.size()));
        (*trainer)(d);
    }
    void map(const float* img, float* dist, uint32_t* rot) override
    {
        Data<DL, float> d(img_layout, std::vector<float>(img, img + img_layout.size()));
        auto r = (*mapper)(d);
        std::memcpy(dist, std::get<0>(r).data(), std::get<0>(r).size() * sizeof(float));
        std::memcpy(rot, std::get<1>(r).data(), std::get<1>(r).size() * sizeof(uint32_t));
    }
    float* som_data() override { return som.get_data_pointer(); }
    size_t som_size() override { return som.size(); }
    void counts(uint32_t* out) override
    {
        auto info = trainer->get_update_info();
        for (uint32_t i = 0; i < info.size(); ++i) out[i] = info[i];
    }
};

} // namespace

extern "C" {

// som_layout: 0 cartesian-2d (s0 x s1), 1 hexagonal (side s0).  C == 0 selects
// the 2-D data layout (one channel, CartesianLayout<2>); C >= 1 selects
// CartesianLayout<3> with C channels.
// shape: 0 quadratic, 1 circular distance region.
void* ref_session_create_shape(const float* som, int som_layout, uint32_t s0, uint32_t s1, uint32_t C, uint32_t id,
    uint32_t nd, uint32_t ed, uint32_t R, int flip, int func, float p0, float p1, float max_dist, int for_map, int shape)
{
    try {
        if (som_layout == 0 && C == 0) return new SessionT<CartesianLayout<2>, CartesianLayout<2>>(som, s0, s1, 1, id, nd, ed, R, flip, func, p0, p1, max_dist, for_map, shape);
        if (som_layout == 0) return new SessionT<CartesianLayout<2>, CartesianLayout<3>>(som, s0, s1, C, id, nd, ed, R, flip, func, p0, p1, max_dist, for_map, shape);
        if (C == 0) return new SessionT<HexagonalLayout, CartesianLayout<2>>(som, s0, s1, 1, id, nd, ed, R, flip, func, p0, p1, max_dist, for_map, shape);
        return new SessionT<HexagonalLayout, CartesianLayout<3>>(som, s0, s1, C, id, nd, ed, R, flip, func, p0, p1, max_dist, for_map, shape);
    } catch (std::exception const&) {
        return nullptr;
    }
}
void* ref_session_create(const float* som, int som_layout, uint32_t s0, uint32_t s1, uint32_t C, uint32_t id,
    uint32_t nd, uint32_t ed, uint32_t R, int flip, int func, float p0, float p1, float max_dist, int for_map)
{
    return ref_session_create_shape(som, som_layout, s0, s1, C, id, nd, ed, R, flip, func, p0, p1, max_dist, for_map, 0);
}
void ref_session_train(void* s, const float* images, uint64_t n, uint64_t image_size)
{
    for (uint64_t i = 0; i < n; ++i) static_cast<Session*>(s)->train(images + i * image_size);
}
void ref_session_map(void* s, const float* images, uint64_t n, uint64_t image_size, uint64_t N, float* dist, uint32_t* rot)
{
    for (uint64_t i = 0; i < n; ++i) static_cast<Session*>(s)->map(images + i * image_size, dist + i * N, rot + i * N);
}
void ref_session_get_som(void* s, float* out)
{
    Session* p = static_cast<Session*>(s);
    std::memcpy(out, p->som_data(), p->som_size() * sizeof(float));
}
void ref_session_get_counts(void* s, uint32_t* out) { static_cast<Session*>(s)->counts(out); }
void ref_session_destroy(void* s) { delete static_cast<Session*>(s); }

// Order in which the reference's shuffled iterator (SelfOrganizingMapLib/DataIteratorShuffled.h) presents
// the n entries of a data file: built on an in-memory file whose entry i holds the value i.
void ref_shuffled_order(uint32_t n, uint64_t seed, int shuffle, uint32_t* out)
{
    std::stringstream ss;
    int header[7] = {2, 0, 0, (int)n, 0, 1, 1};
    ss.write(reinterpret_cast<const char*>(header), sizeof(header));
    for (uint32_t i = 0; i < n; ++i) { float v = (float)i; ss.write(reinterpret_cast<const char*>(&v), sizeof(float)); }
    auto cur = DataIteratorShuffled<CartesianLayout<1>, float>(ss, seed, shuffle != 0);
    auto end = DataIteratorShuffled<CartesianLayout<1>, float>(ss, true);
    for (uint32_t k = 0; cur != end && k < n; ++cur, ++k) out[k] = (uint32_t)(*cur)[0];
}

// Rotation set through the reference's SpatialTransformer (C == 0: 2-D layout).
void ref_rotation_set(const float* img, uint32_t C, uint32_t id, uint32_t nd, uint32_t R, int flip, float* out)
{
    if (C == 0) {
        Data<CartesianLayout<2>, float> d(CartesianLayout<2>{{id, id}}, std::vector<float>(img, img + (size_t)id * id));
        auto r = SpatialTransformer<CartesianLayout<2>>()(d, R, flip, Interpolation::BILINEAR, CartesianLayout<2>{{nd, nd}});
        std::memcpy(out, r.data(), r.size() * sizeof(float));
    } else {
        Data<CartesianLayout<3>, float> d(CartesianLayout<3>{{C, id, id}}, std::vector<float>(img, img + (size_t)C * id * id));
        auto r = SpatialTransformer<CartesianLayout<3>>()(d, R, flip, Interpolation::BILINEAR, CartesianLayout<3>{{C, nd, nd}});
        std::memcpy(out, r.data(), r.size() * sizeof(float));
    }
}

// Integer-typed instantiations used by the reference's own unit tests.
void ref_rotation_set_int(const int* img, uint32_t C, uint32_t id, uint32_t nd, uint32_t R, int flip, int* out)
{
    if (C == 0) {
        Data<CartesianLayout<2>, int> d(CartesianLayout<2>{{id, id}}, std::vector<int>(img, img + (size_t)id * id));
        auto r = SpatialTransformer<CartesianLayout<2>>()(d, R, flip, Interpolation::BILINEAR, CartesianLayout<2>{{nd, nd}});
        std::memcpy(out, r.data(), r.size() * sizeof(int));
    } else {
        Data<CartesianLayout<3>, int> d(CartesianLayout<3>{{C, id, id}}, std::vector<int>(img, img + (size_t)C * id * id));
        auto r = SpatialTransformer<CartesianLayout<3>>()(d, R, flip, Interpolation::BILINEAR, CartesianLayout<3>{{C, nd, nd}});
        std::memcpy(out, r.data(), r.size() * sizeof(int));
    }
}

float ref_distance_pair(const float* a, const float* b, uint32_t C, uint32_t nd, uint32_t ed)
{
    if (C == 0) return EuclideanDistanceFunctor<CartesianLayout<2>>()(a, b, CartesianLayout<2>{{nd, nd}}, ed);
    return EuclideanDistanceFunctor<CartesianLayout<3>>()(a, b, CartesianLayout<3>{{C, nd, nd}}, ed);
}

void ref_update_factors(int som_layout, uint32_t s0, uint32_t s1, int func, float p0, float p1, float max_dist, float* F)
{
    auto f = make_func(func, p0, p1);
    if (som_layout == 0) {
        CartesianLayout<2> l{{s0, s1}};
        uint32_t N = l.size();
        for (uint32_t i = 0; i < N; ++i) for (uint32_t j = 0; j < N; ++j) {
            float d = l.get_distance(i, j);
            F[(size_t)i * N + j] = (max_dist <= 0 || d < max_dist) ? f(d) : 0.0f;
        }
    } else {
        HexagonalLayout l({s0, s0});
        uint32_t N = l.size();
        for (uint32_t i = 0; i < N; ++i) for (uint32_t j = 0; j < N; ++j) {
            float d = l.get_distance(i, j);
            F[(size_t)i * N + j] = (max_dist <= 0 || d < max_dist) ? f(d) : 0.0f;
        }
    }
}

void ref_update_factors_3d(uint32_t s0, uint32_t s1, uint32_t s2, int func, float p0, float p1, float max_dist, float* F)
{
    auto f = make_func(func, p0, p1);
    CartesianLayout<3> l{{s0, s1, s2}};
    uint32_t N = l.size();
    for (uint32_t i = 0; i < N; ++i) for (uint32_t j = 0; j < N; ++j) {
        float d = l.get_distance(i, j);
        F[(size_t)i * N + j] = (max_dist <= 0 || d < max_dist) ? f(d) : 0.0f;
    }
}

void ref_fill_random_uniform(float* a, uint64_t n, uint32_t seed) { fill_random_uniform(a, n, seed); }

int ref_num_threads() { return omp_get_max_threads(); }

// Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; a timed baseline sets its thread count itself.
void ref_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }

} // extern "C"
